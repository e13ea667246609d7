/*
 * CPU oracle for the quantized-matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's W4A16 /
 * W4A8 int4 linear and of its MXFP4 mixture-of-experts operator.  It is the
 * checker for the CUDA kernels: only the test-suite, the smoke check and the
 * benchmark's cpu_baseline leg may call it.  Nothing under garnet_b200/ links,
 * imports or executes it.
 *
 * Pinning: int4 functions are compared bit-for-bit with the reference's own
 * compiled sources (oracle/_ref, built by oracle/Makefile) and with the golden
 * vectors under tests/golden/; the MoE functions are compared with golden
 * input/output pairs captured from the reference's pure-Python MoE
 * (test2026/gpt_oss/make_fixture.py) and with the 256 x 16 MXFP4 decode table
 * property of test2026/gpt_oss/kernel_parity.cpp:537-559.
 *
 * Each function cites the reference file:line whose arithmetic it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- helpers */

/* Round-to-nearest-even to bf16, returned as fp32.
 * test2026/gpt_oss/kernel_parity.cpp:20 (host twin of gpt_oss_kernels.cu:16). */
static inline float bf(float x)
{
    uint32_t v;
    memcpy(&v, &x, 4);
    if ((v & 0x7fffffffu) > 0x7f800000u) {          /* NaN stays NaN */
        v |= 0x00400000u;
        v &= 0xffff0000u;
    } else {
        v += 0x7fffu + ((v >> 16) & 1u);
        v &= 0xffff0000u;
    }
    memcpy(&x, &v, 4);
    return x;
}

ORC_API float orc_bf16_round(float x) { return bf(x); }

ORC_API int orc_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* IEEE binary16 round-to-nearest-even, as src/model/weight_quantization.cpp:58-107. */
static uint16_t float_to_fp16(float value)
{
    uint32_t bits;
    memcpy(&bits, &value, 4);
    const uint32_t sign = (bits >> 16) & 0x8000u;
    const uint32_t mag = bits & 0x7fffffffu;
    if (mag >= 0x7f800000u) return (uint16_t)(sign | (mag > 0x7f800000u ? 0x7e00u : 0x7c00u));
    int e = (int)(mag >> 23) - 127;
    uint32_t m = mag & 0x7fffffu;
    if (e > 15) return (uint16_t)(sign | 0x7c00u);
    if (e < -14) {
        if (e < -24) return (uint16_t)sign;
        m |= 0x800000u;
        const int sh = -e - 14 + 13;
        uint32_t r = m >> sh;
        const uint32_t rem = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (r & 1u))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t r = m >> 13;
    const uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) {
        ++r;
        if (r == 0x400u) { r = 0; if (++e > 15) return (uint16_t)(sign | 0x7c00u); }
    }
    return (uint16_t)(sign | ((uint32_t)(e + 15) << 10) | r);
}

/* src/model/weight_quantization.cpp:23-56. */
static float fp16_to_float(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu, bits;
    if (e == 0) {
        if (m == 0) bits = sign;
        else {
            int sh = 0;
            while (!(m & 0x400u)) { m <<= 1; ++sh; }
            m &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - sh) << 23) | (m << 13);
        }
    } else if (e == 0x1fu) bits = sign | 0x7f800000u | (m << 13);
    else bits = sign | ((e + 112u) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

ORC_API uint16_t orc_float_to_fp16(float v) { return float_to_fp16(v); }
ORC_API float orc_fp16_to_float(uint16_t h) { return fp16_to_float(h); }

/* Canonical int4 element: two's-complement nibble `index&1` of byte `index/2`.
 * test2026/native/weight_quantization_test.cpp:47-53 (Unpack). */
static inline int int4_at(const uint8_t* packed, size_t index)
{
    const int v = (packed[index >> 1] >> ((index & 1u) * 4u)) & 15;
    return v >= 8 ? v - 16 : v;
}

/* ------------------------------------------------------------ int4 linear */

/* Symmetric per-(row, K-block) int4 quantizer.
 * src/model/weight_quantization.cpp:188-270: scale = max(-min/8, max/7) with
 * min,max starting at 0; non-finite or non-positive scale -> 1; the scale is
 * stored rounded (fp16 in the reference; `scale_kind` 1 selects bf16, the
 * format the B200 path is specified with) and the quantized value is
 * clamp(nearbyint(v / stored_scale), -8, 7).  Returns the maximum absolute
 * reconstruction error like QuantizedWeight::maximumAbsoluteError. */
ORC_API double orc_int4_quantize(const float* w, long rows, long cols, int block,
                                 int scale_kind, uint8_t* packed, uint16_t* scales)
{
    const long groups = cols / block;
    double worst = 0.0;
    memset(packed, 0, (size_t)((rows * cols + 1) / 2));
    for (long r = 0; r < rows; ++r)
        for (long g = 0; g < groups; ++g) {
            const size_t start = (size_t)r * cols + (size_t)g * block;
            float lo = 0.f, hi = 0.f;
            for (int o = 0; o < block; ++o) {
                const float v = w[start + o];
                lo = fminf(lo, v);
                hi = fmaxf(hi, v);
            }
            float scale = fmaxf(-lo / 8.0f, hi / 7.0f);
            if (!isfinite(scale) || scale <= 0.f) scale = 1.0f;
            uint16_t sbits;
            float stored;
            if (scale_kind == 0) { sbits = float_to_fp16(scale); stored = fp16_to_float(sbits); }
            else {
                stored = bf(scale);
                uint32_t u;
                memcpy(&u, &stored, 4);
                sbits = (uint16_t)(u >> 16);
            }
            scales[r * groups + g] = sbits;
            for (int o = 0; o < block; ++o) {
                const size_t i = start + o;
                int q = (int)nearbyintf(w[i] / stored);
                q = q < -8 ? -8 : (q > 7 ? 7 : q);
                packed[i >> 1] |= (uint8_t)((q & 15) << ((i & 1u) * 4u));
                const double err = fabs((double)(w[i] - (float)q * stored));
                if (err > worst) worst = err;
            }
        }
    return worst;
}

/* Dequantised weights q * s as fp32 (exact: |q| <= 8 and s has <= 11
 * significant bits).  weight_quantization_test.cpp:47-53 times the scale. */
ORC_API void orc_int4_dequant(const uint8_t* packed, const float* scales, long rows,
                              long cols, int block, float* out)
{
    const long groups = cols / block;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        for (long c = 0; c < cols; ++c)
            out[(size_t)r * cols + c] =
                (float)int4_at(packed, (size_t)r * cols + c) * scales[r * groups + c / block];
}

/* Exact W4A16 product: y[m,n] = sum_k x[m,k] * (q[n,k] * s[n,k/block]),
 * accumulated in index order in fp32 (y32) and fp64 (y64, may be NULL).
 * x is expected to hold bf16-representable values.  No output rounding here;
 * callers round to bf16 when they compare with the device result. */
ORC_API void orc_w4a16_exact(const uint8_t* packed, const float* scales, long N, long K,
                             int block, const float* x, long M, float* y32, double* y64)
{
    const long groups = K / block;
#pragma omp parallel for schedule(static)
    for (long n = 0; n < N; ++n)
        for (long m = 0; m < M; ++m) {
            float a32 = 0.f;
            double a64 = 0.0;
            for (long k = 0; k < K; ++k) {
                const float w = (float)int4_at(packed, (size_t)n * K + k) * scales[n * groups + k / block];
                a32 += x[m * K + k] * w;
                a64 += (double)x[m * K + k] * (double)w;
            }
            y32[m * N + n] = a32;
            if (y64) y64[m * N + n] = a64;
        }
}

/* The reference CPU operator (W4A8): per K-group the activation is quantised to
 * int8 with scale max|x|/127 (1 when the group is all zero), the dot product is
 * an exact integer, and y[n] = sum_g float(dot) * s_x[g] * s_w[n,g] in fp32.
 * src/backends/cpu/q4q8_linear.cpp:346-383.  DotGroup's biased-nibble form
 * (sum (q+8)*qx - 8*sum qx, :146-171,:377) equals sum q*qx exactly in int32,
 * which is what is computed here.  `threads` <= 1 runs single-threaded. */
ORC_API void orc_q4q8_forward(const uint8_t* packed, const float* scales, long N, long K,
                              int block, const float* x, float* y, int threads)
{
    const long groups = K / block;
    int8_t* qx = (int8_t*)malloc((size_t)K);
    float* sx = (float*)malloc(sizeof(float) * (size_t)groups);
    for (long g = 0; g < groups; ++g) {
        const float* xg = x + g * block;
        float amax = 0.f;
        for (int i = 0; i < block; ++i) amax = fmaxf(amax, fabsf(xg[i]));
        const float s = amax > 0.f ? amax / 127.0f : 1.0f;
        const float inv = 1.0f / s;
        sx[g] = s;
        for (int i = 0; i < block; ++i) {
            int v = (int)nearbyintf(xg[i] * inv);
            v = v < -127 ? -127 : (v > 127 ? 127 : v);
            qx[g * block + i] = (int8_t)v;
        }
    }
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
    for (long n = 0; n < N; ++n) {
        float value = 0.f;
        const uint8_t* row = packed + (size_t)n * K / 2;
        for (long g = 0; g < groups; ++g) {
            int dot = 0;
            const uint8_t* p = row + g * block / 2;
            const int8_t* a = qx + g * block;
            for (int i = 0; i < block; i += 2) {
                const int b = p[i >> 1];
                const int lo = ((b & 15) ^ 8) - 8, hi = ((b >> 4) ^ 8) - 8;
                dot += lo * a[i] + hi * a[i + 1];
            }
            /* The reference builds this file with -mfma and the compiler's default
             * contraction (CMakeLists.txt:389-394), so the last multiply and the add
             * fuse; fmaf() states that explicitly. */
            value = fmaf((float)dot * sx[g], scales[n * groups + g], value);
        }
        y[n] = value;
    }
    free(qx);
    free(sx);
}

/* ------------------------------------------------------------------ MXFP4 */

/* One MXFP4 element: +-{0,.5,1,1.5,2,3,4,6}[code&7] * 2^(e8m0-127); the bits are
 * built directly, covering subnormal results, overflow to infinity and e8m0
 * 255 = NaN.  plugins/gpt_oss/cuda/gpt_oss_kernels.cu:50-70. */
static float mxfp4_bits(int code, int exponent)
{
    if (exponent == 255) return NAN;
    const uint32_t sign = (uint32_t)(code & 8) << 28;
    const int mag = code & 7;
    uint32_t bits;
    if (!mag) bits = sign;
    else {
        const int adj = exponent + (mag >> 1) - 1;
        const uint32_t man = (mag >= 3 && (mag & 1)) ? 0x00400000u : 0u;
        if (adj >= 255) bits = sign | 0x7f800000u;
        else if (adj > 0) bits = sign | ((uint32_t)adj << 23) | man;
        else bits = sign | ((0x00800000u | man) >> (1 - adj));
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Host twin used by the reference's own CPU oracle:
 * bf(ldexp(lut[code], e-127)).  test2026/gpt_oss/kernel_parity.cpp:531-535. */
static float mxfp4_ldexp(int code, int exponent)
{
    static const float lut[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float v = (code & 8) ? -lut[code & 7] : lut[code & 7];
    return bf(ldexpf(v, exponent - 127));
}

ORC_API float orc_mxfp4_value(int code, int exponent) { return mxfp4_bits(code, exponent); }
ORC_API float orc_mxfp4_value_ldexp(int code, int exponent) { return mxfp4_ldexp(code, exponent); }

/* Element (row, col) of an original-layout MXFP4 matrix: byte col/2 of the row
 * (low nibble = even column), one scale byte per 32 columns.
 * gpt_oss_kernels.cu:50-54. */
static float g_mxfp4_table[256][16];
__attribute__((constructor)) static void mxfp4_table_init(void)
{
    for (int e = 0; e < 256; ++e)
        for (int c = 0; c < 16; ++c) g_mxfp4_table[e][c] = mxfp4_bits(c, e);
}

static inline float mxfp4_at(const uint8_t* blocks, const uint8_t* scales, size_t row,
                             long col, long width)
{
    const uint8_t b = blocks[row * (size_t)(width / 2) + (size_t)(col / 2)];
    const int code = (col & 1) ? b >> 4 : b & 15;
    return g_mxfp4_table[scales[row * (size_t)(width / 32) + (size_t)(col / 32)]][code];
}

ORC_API void orc_mxfp4_dequant(const uint8_t* blocks, const uint8_t* scales, long rows,
                               long width, float* out)
{
#pragma omp parallel for schedule(static)
    for (long r = 0; r < rows; ++r)
        for (long c = 0; c < width; ++c)
            out[(size_t)r * width + c] = mxfp4_at(blocks, scales, (size_t)r, c, width);
}

/* Router: logits[t,e] = bf(sum_d x[t,d]*W[e,d] + b[e]) (fp32, index order), then
 * k rounds of arg-max with ties to the lowest expert index, and
 * p[j] = bf(exp(l_j - l_0) / sum_{i<k} exp(l_i - l_0)) over the selected logits.
 * kernel_parity.cpp:627-633; gpt_oss_kernels.cu:537-587, :681-726.
 * `logits` receives the rounded logits (may be NULL). */
ORC_API void orc_moe_route(const float* x, const float* router_w, const float* router_b,
                           long tokens, int hidden, int experts, int topk, float* logits,
                           int32_t* selected, float* probs)
{
#pragma omp parallel for schedule(static)
    for (long t = 0; t < tokens; ++t) {
        float* l = (float*)malloc(sizeof(float) * (size_t)experts);
        char* used = (char*)calloc((size_t)experts, 1);
        for (int e = 0; e < experts; ++e) {
            float v = 0.f;
            for (int d = 0; d < hidden; ++d) v += x[t * hidden + d] * router_w[(size_t)e * hidden + d];
            l[e] = bf(v + router_b[e]);
            if (logits) logits[t * experts + e] = l[e];
        }
        float top[64];
        for (int j = 0; j < topk; ++j) {
            int best = -1;
            for (int e = 0; e < experts; ++e)
                if (!used[e] && (best < 0 || l[e] > l[best])) best = e;
            if (best < 0) best = 0;
            used[best] = 1;
            selected[t * topk + j] = best;
            top[j] = l[best];
        }
        float total = 0.f;
        for (int j = 0; j < topk; ++j) total += expf(top[j] - top[0]);
        for (int j = 0; j < topk; ++j) probs[t * topk + j] = bf(expf(top[j] - top[0]) / total);
        free(l);
        free(used);
    }
}

/* Experts for a given routing.  Per routed slot (router order j = 0..k-1):
 *   g = min(bf(bf(sum x*w_gate) + b[2i]), limit)
 *   u = clamp(bf(bf(sum x*w_up) + b[2i+1]), -limit, limit)
 *   h_i = bf(bf(g * bf(1/(1+exp(-bf(1.702 g))))) * bf(u + 1))
 *   o[d] += bf(bf(sum_i h_i*w_down[d,i]) + bd[d]) * p_j
 * and finally o = bf(o) unless `round_output` is 0 (the per-rank partial of an
 * expert-sharded run is left unrounded, gpt_oss_kernels.cu:810).  Gate and up
 * rows are interleaved (row 2i = gate_i, row 2i+1 = up_i).
 * kernel_parity.cpp:634-647; gpt_oss_kernels.cu:762-811.
 * An expert e is computed only when expert_lo <= e < expert_hi and, if
 * `modulo` > 0, e % modulo == residue (the reference's 2-way rule is modulo 2,
 * gpt_oss_kernels.cu:771).
 * `mass` (may be NULL) receives sum_j |bf(bf(v)+bd)| * p_j, the scale of the
 * summands, against which errors of outputs that nearly cancel are judged. */
ORC_API void orc_moe_experts(const float* x, const int32_t* selected, const float* probs,
                             const uint8_t* gu_blocks, const uint8_t* gu_scales,
                             const float* gu_bias, const uint8_t* dn_blocks,
                             const uint8_t* dn_scales, const float* dn_bias, long tokens,
                             int hidden, int inter, int experts, int topk, float limit,
                             int expert_lo, int expert_hi, int modulo, int residue,
                             int round_output, float* y, float* mass)
{
    (void)experts;
#pragma omp parallel for schedule(dynamic, 1)
    for (long t = 0; t < tokens; ++t) {
        float* h = (float*)malloc(sizeof(float) * (size_t)inter);
        float* o = (float*)calloc((size_t)hidden, sizeof(float));
        float* ms = (float*)calloc((size_t)hidden, sizeof(float));
        const float* xt = x + t * hidden;
        for (int j = 0; j < topk; ++j) {
            const int e = selected[t * topk + j];
            if (e < expert_lo || e >= expert_hi) continue;
            if (modulo > 0 && e % modulo != residue) continue;
            const float p = probs[t * topk + j];
            for (int i = 0; i < inter; ++i) {
                const size_t row = (size_t)e * 2 * inter + 2 * (size_t)i;
                float g = 0.f, u = 0.f;
                for (int d = 0; d < hidden; ++d) {
                    g += xt[d] * mxfp4_at(gu_blocks, gu_scales, row, d, hidden);
                    u += xt[d] * mxfp4_at(gu_blocks, gu_scales, row + 1, d, hidden);
                }
                g = fminf(bf(bf(g) + gu_bias[row]), limit);
                u = fminf(limit, fmaxf(-limit, bf(bf(u) + gu_bias[row + 1])));
                const float glu = bf(g * bf(1.f / (1.f + expf(-bf(1.702f * g)))));
                h[i] = bf(glu * bf(u + 1.f));
            }
            for (int d = 0; d < hidden; ++d) {
                const size_t row = (size_t)e * hidden + (size_t)d;
                float v = 0.f;
                for (int i = 0; i < inter; ++i) v += h[i] * mxfp4_at(dn_blocks, dn_scales, row, i, inter);
                const float val = bf(bf(v) + dn_bias[row]);
                o[d] += val * p;
                ms[d] += fabsf(val) * p;
            }
        }
        for (int d = 0; d < hidden; ++d) y[t * hidden + d] = round_output ? bf(o[d]) : o[d];
        if (mass)
            for (int d = 0; d < hidden; ++d) mass[t * hidden + d] = ms[d];
        free(h);
        free(o);
        free(ms);
    }
}

/* The two halves of the expert computation on already routed rows, one expert per
 * row (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:762-811: gateUp, then down):
 *   hidden[r, i] = bf( bf( g * bf(sigmoid(bf(1.702 g))) ) * bf(u + 1) ),
 *                  g = min(bf(bf(x . w_gate_i) + b), limit), u = clamp(bf(bf(x . w_up_i) + b), +-limit);
 *   vals[r, d]   = bf( bf(hidden[r, :] . w_down_d) + b_down_d ).
 * Checking them separately keeps a one-step difference in a bf16 rounding of the
 * first half (legitimate: it depends on the fp32 summation order) from being
 * amplified by the second. */
ORC_API void orc_moe_rows_hidden(const float* x, const int32_t* row_expert, const uint8_t* gu_blocks,
                                 const uint8_t* gu_scales, const float* gu_bias, long rows, int hidden,
                                 int inter, float limit, float* out)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (long r = 0; r < rows; ++r) {
        const int e = row_expert[r];
        const float* xt = x + r * hidden;
        for (int i = 0; i < inter; ++i) {
            const size_t row = (size_t)e * 2 * inter + 2 * (size_t)i;
            float g = 0.f, u = 0.f;
            for (int d = 0; d < hidden; ++d) {
                g += xt[d] * mxfp4_at(gu_blocks, gu_scales, row, d, hidden);
                u += xt[d] * mxfp4_at(gu_blocks, gu_scales, row + 1, d, hidden);
            }
            g = fminf(bf(bf(g) + gu_bias[row]), limit);
            u = fminf(limit, fmaxf(-limit, bf(bf(u) + gu_bias[row + 1])));
            const float glu = bf(g * bf(1.f / (1.f + expf(-bf(1.702f * g)))));
            out[r * inter + i] = bf(glu * bf(u + 1.f));
        }
    }
}

ORC_API void orc_moe_rows_down(const float* h, const int32_t* row_expert, const uint8_t* dn_blocks,
                               const uint8_t* dn_scales, const float* dn_bias, long rows, int hidden,
                               int inter, float* out)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (long r = 0; r < rows; ++r) {
        const int e = row_expert[r];
        const float* hr = h + r * inter;
        for (int d = 0; d < hidden; ++d) {
            const size_t row = (size_t)e * hidden + (size_t)d;
            float v = 0.f;
            for (int i = 0; i < inter; ++i) v += hr[i] * mxfp4_at(dn_blocks, dn_scales, row, i, inter);
            out[r * hidden + d] = bf(bf(v) + dn_bias[row]);
        }
    }
}

