/*
 * garnet_b200.h - C ABI of the B200 (sm_100a) quantized-matmul library.
 *
 * Drop-in boundary for the two quantized operators of Garnet:
 *   - the weight-only int4 linear (every Qwen3 decoder projection and lm_head);
 *   - the gpt-oss MXFP4 mixture-of-experts operator `gpt_oss_moe_mxfp4`.
 * Every entry point takes plain pointers, sizes and a CUDA stream (passed as
 * void*), returns an int status and never throws.  Each declaration cites the
 * reference interface it replaces (path inside the Garnet checkout : line).
 *
 * Ownership: the caller owns inputs, outputs, workspaces and the stream.  A
 * handle owns only its repacked weight copy and a few counters.  `*_run`
 * functions do not allocate, free or synchronise.  A handle is not thread-safe:
 * use one handle per (device, stream), as the reference requires of its plugin
 * objects (plugins/gpt_oss/include/gpt_oss_marlin.h:14-16).
 */
#ifndef GARNET_B200_H
#define GARNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GARNET_B200_ABI 1

/* Status codes.  The reference returns cudaError_t from its free functions and
 * int (0 = ok) from its C exports (src/include/garnet_serving.h:22-36); here
 * cudaErrorInvalidValue maps to INVALID_VALUE and cudaErrorNotSupported ("use
 * the fallback", plugins/gpt_oss/tensorrt/gpt_oss_plugin.cpp:405) to
 * NOT_SUPPORTED. */
enum {
    GARNET_B200_OK = 0,
    GARNET_B200_INVALID_VALUE = 1,
    GARNET_B200_NOT_SUPPORTED = 2,
    GARNET_B200_CUDA_ERROR = 3,
    GARNET_B200_DEVICE_FAULT = 4,   /* a bounded device-side wait gave up */
    GARNET_B200_OUT_OF_MEMORY = 5
};

enum { GARNET_B200_FP16 = 0, GARNET_B200_BF16 = 1, GARNET_B200_FP32 = 2 };

/* Thread-local text of the last failure on the calling thread. */
const char* garnet_b200_last_error(void);

/* ---- plugin discovery -------------------------------------------------------
 * Replaces the four callbacks of GarnetOperatorModuleBridge
 * (src/model/operator_module_bridge.h:6-14): abi, manifest(), resolve_callback(name),
 * binary_path().  The manifest has the keys of the reference's manifest
 * (plugins/gpt_oss/tensorrt/gpt_oss_plugin.cpp:497-503): id, module, abi, version,
 * backend, operators. */
int garnet_b200_abi_version(void);
const char* garnet_b200_manifest_json(void);
void* garnet_b200_resolve(const char* symbol_name);
const char* garnet_b200_binary_path(void);

/* Which checkpoint tensors the int4 path quantizes: rank 2, positive extents, K a
 * multiple of the block, dtype "BF16", "F16" or "F32", and a name that ends in one of
 * the Qwen projection names (q/k/v/o_proj, the linear-attention projections,
 * gate/up/down_proj, lm_head).  Returns 1 or 0.  Host only.  Replaces
 * Garnet::IsQwenLinearWeightForINT4 (src/model/weight_quantization.cpp:146-186);
 * `dtype`, `rank` and `shape` are the fields of SafeTensorMetadata it reads. */
int garnet_b200_is_int4_linear_weight(const char* name, const char* dtype, int rank, const int64_t* shape, int block);

/* Launches one warp that waits, with a limit of `limit_ms` (1..2000), on a barrier
 * that nothing ever completes, synchronises `stream` and returns DEVICE_FAULT: the way
 * every bounded device-side wait of this library ends when its partner never shows
 * up, without hanging or faulting the GPU.  The context stays usable.  For tests of
 * the fault reporting; the reference reports such waits through a fault word as well
 * (plugins/gpt_oss/cuda/tp_peer_owner.cuh:40-46,308-315). */
int garnet_b200_selftest_bounded_wait(int limit_ms, void* stream);

/* ---- int4 quantizer ---------------------------------------------------------
 * Replaces Garnet::QuantizeSymmetricINT4 (src/model/weight_quantization.cpp:188-270)
 * for a device-resident weight: per (row, K-group) scale = max(-min/8, max/7),
 * stored rounded to `scale_dtype` (the reference stores fp16; the B200 path is
 * specified with bf16), q = clamp(nearbyint(v / stored_scale), -8, 7), canonical
 * nibble packing.  `d_src` is [rows, cols] of `src_dtype`; `d_nibbles` receives
 * rows*cols/2 bytes, `d_scales` rows*cols/group 16-bit values. */
int garnet_b200_int4_quantize(const void* d_src, int src_dtype, int64_t rows, int64_t cols, int group,
                              int scale_dtype, uint8_t* d_nibbles, uint16_t* d_scales, void* stream);

/* ---- W4A16 linear -----------------------------------------------------------
 * y[M,N] = x[M,K] * W^T with W int4 (group scales), x and y bf16, fp32
 * accumulation.  Replaces, for the CUDA backend, the int4 branch of
 * GetOrCreateTRTWeight + MatMul (src/backends/tensorrt/trt_builder.cpp:3285-3344,
 * :7398-7408) and mirrors the life cycle of the CPU operator Garnet::Q4Q8Linear
 * (src/backends/cpu/q4q8_linear.h:21-35): Prepare -> create, Forward -> run. */
typedef struct garnet_b200_w4a16* garnet_b200_w4a16_t;

/* Bytes of the packed form of an [N,K] matrix (codes and scales together). */
int garnet_b200_w4a16_packed_bytes(int n, int k, int group, size_t* bytes);

/* Host repacker: canonical nibbles + 16-bit scales -> packed bytes, identical to
 * what the device repacker writes.  Counterpart of the reference's host packers
 * that let an engine hold prepacked constants (Q4Q8Linear::Prepare,
 * q4q8_linear.cpp:227-283; PackGptOssMarlinWeight, gpt_oss_marlin_pack.h:74-193). */
int garnet_b200_w4a16_pack_host(const uint8_t* nibbles, const uint16_t* scales, int scale_dtype, int n, int k,
                                int group, uint8_t* packed);

/* Creates the operator from device-resident canonical weights.  With
 * shard_world > 1 the handle keeps only rows [rank*N/world, (rank+1)*N/world)
 * (tensor-parallel split along N; the reference's vocab-parallel lm_head,
 * trt_builder.cpp:7360-7371).  Repacks on `stream` and synchronises it once.
 * Q4Q8Linear::Prepare (q4q8_linear.cpp:227). */
int garnet_b200_w4a16_create(const uint8_t* d_nibbles, const void* d_scales, int scale_dtype, int n, int k,
                             int group, int shard_rank, int shard_world, void* stream,
                             garnet_b200_w4a16_t* out);

/* The same with the split along K: the handle keeps columns [rank*K/world, (rank+1)*K/world)
 * of every row (K/world a multiple of `group`), `run` takes x[m, K/world] - this rank's
 * columns of the activations - and returns the rank's partial sums y[m, N] in bf16, to be
 * added over the ranks (garnet_b200_comm_all_reduce_bf16).  The reference's row-parallel
 * projections (tp_mode "row": the weight sliced along axis 1,
 * src/backends/tensorrt/trt_builder.cpp:7347-7359, followed by GptOssTpAllReduceBf16). */
int garnet_b200_w4a16_create_k_shard(const uint8_t* d_nibbles, const void* d_scales, int scale_dtype, int n, int k,
                                     int group, int shard_rank, int shard_world, void* stream,
                                     garnet_b200_w4a16_t* out);

/* Creates the operator over already packed device bytes, which are borrowed, not
 * copied (Q4Q8Linear::BindPackedView, q4q8_linear.cpp:285-313). */
int garnet_b200_w4a16_create_prepacked(const uint8_t* d_packed, int scale_dtype, int n, int k, int group,
                                       garnet_b200_w4a16_t* out);

/* Logical rows held by this handle (N / shard_world) and K. */
int garnet_b200_w4a16_shape(garnet_b200_w4a16_t h, int* n_local, int* k);

/* Workspace bytes `run` needs for a batch of m rows (0 is possible). */
int garnet_b200_w4a16_workspace(garnet_b200_w4a16_t h, int m, size_t* bytes);

/* y[m, n_local] = x[m, k] W^T.  x, y bf16 device pointers, row-major, 16-byte
 * aligned.  Q4Q8Linear::Forward (q4q8_linear.cpp:315-389).  `flags`: bit 0 asks
 * for a programmatic dependent launch, so that this kernel's weight prefetch
 * overlaps the tail of the previous kernel in the stream.  Up to 16 rows (8 when
 * K > 4096) take the streaming kernel: exact integer sums per group of 15-bit block
 * fixed-point activations; more rows take the tensor-core tile kernel, which multiplies
 * by the weights rounded once to bf16. */
int garnet_b200_w4a16_run(garnet_b200_w4a16_t h, const void* d_x, void* d_y, int m, void* d_workspace,
                          size_t workspace_bytes, unsigned flags, void* stream);

/* Up to 4 linears that read the same x (same K), one launch: y_g[m, n_g] = x W_g^T.
 * The device form of the reference's packed projections, which concatenate q/k/v and
 * gate/up along N because they share their input (qwen3_text_qkv_packed,
 * qwen3_mlp_gate_up_swiglu_packed: src/backends/tensorrt/trt_builder.cpp:7565-7577,
 * :7727-7738), without requiring the weights to be stored concatenated. */
int garnet_b200_w4a16_run_group(const garnet_b200_w4a16_t* handles, int count, const void* d_x, void* const* d_ys,
                                int m, unsigned flags, void* stream);

/* A prepared list of linears that one persistent launch runs back to back: linear i
 * computes d_ys[i][m, n_i] = d_xs[i][m, k_i] W_i^T, every linear with the same batch m
 * (at most 16, less for very large K).  deps[i] is -1, or the index of an EARLIER
 * linear whose output d_xs[i] holds (directly, or through work of the caller's that
 * the list does not see is not supported: the list only orders its own linears);
 * linear i then reads its x only after that linear has completed on every SM.
 * deps may be NULL (no dependencies).  The weights of later linears stream into
 * shared memory while earlier ones finish, so a decode step pays one launch and no
 * gaps between its projections.  This is the device form of the engine running the
 * captured sequence of isLinear operators of one decode step
 * (src/backends/tensorrt/trt_builder.cpp:7268-7423) with one enqueue.
 * create allocates a small device table and counters; run allocates nothing and does
 * not synchronise (flags as for garnet_b200_w4a16_run).  Pointers are captured at
 * create time.  A list with dependencies needs all of the GPU's SMs for its CTAs to
 * wait on one another: run it on a GPU that no other long-running kernel occupies,
 * one run at a time.  garnet_b200_w4a16_list_fault is non-zero after a bounded
 * device-side wait gave up (as garnet_b200_w4a16_fault). */
typedef struct garnet_b200_w4a16_list_s* garnet_b200_w4a16_list_t;
int garnet_b200_w4a16_list_create(const garnet_b200_w4a16_t* handles, const void* const* d_xs, void* const* d_ys,
                                  const int* deps, int count, int m, garnet_b200_w4a16_list_t* out);
/* The same list with the glue between the linears of a decoder layer folded into them, so that
 * a layer's o_proj, gate/up, down and the next layer's q/k/v are one launch (the reference
 * lowers these as separate TensorRT layers around its linears: RMS norm and packed q/k/v,
 * src/backends/tensorrt/trt_builder.cpp:7565-7726; packed gate/up with SiLU and multiply,
 * :7727-7800; the residual additions of the decoder layer):
 *   d_norm_weight  bf16 [K]: the input rows are first RMS-normalised,
 *                  x' = bf16(x / sqrt(mean(x^2) + norm_eps) * w);
 *   activation 1:  the source rows are [m, 2K] (a packed gate/up output) and the input is
 *                  bf16(silu(source[:, :K]) * source[:, K:]);
 *   d_residual     bf16 [m, N] in memory, or residual_dep = an earlier item of the list whose
 *                  output it is: y = bf16(x' W^T + residual), one rounding.
 * Items are zero-initialised apart from `dep` and `residual_dep`, which are -1 when unused. */
typedef struct garnet_b200_w4a16_list_item {
    garnet_b200_w4a16_t linear;
    const void* d_x;            /* source rows: bf16 [m, K], or [m, 2K] with activation 1 */
    void* d_y;                  /* bf16 [m, N] */
    int dep;                    /* -1, or the earlier item whose d_y is this d_x */
    int activation;             /* 0 or 1 */
    const void* d_norm_weight;  /* NULL or bf16 [K] */
    float norm_eps;
    int residual_dep;           /* -1, or the earlier item whose output is added */
    const void* d_residual;     /* NULL or bf16 [m, N] */
} garnet_b200_w4a16_list_item;
int garnet_b200_w4a16_list_create_ex(const garnet_b200_w4a16_list_item* items, int count, int m,
                                     garnet_b200_w4a16_list_t* out);
int garnet_b200_w4a16_list_run(garnet_b200_w4a16_list_t list, unsigned flags, void* stream);
int garnet_b200_w4a16_list_fault(garnet_b200_w4a16_list_t list);
void garnet_b200_w4a16_list_destroy(garnet_b200_w4a16_list_t list);

/* Same call for host-resident x and y (the plugin-facing form: host -> device
 * copy, kernel, device -> host copy on `stream`, then a stream synchronise).
 * The device staging behind it belongs to the handle and is allocated by
 * garnet_b200_w4a16_reserve_host(h, max_m), once, outside the hot loop; run_host
 * itself allocates nothing and rejects more rows than were reserved. */
int garnet_b200_w4a16_reserve_host(garnet_b200_w4a16_t h, int max_m);
int garnet_b200_w4a16_run_host(garnet_b200_w4a16_t h, const void* h_x, void* h_y, int m, void* stream);
/* The same call without the final synchronisation: x is copied in and the kernel is
 * enqueued on `stream`; y is complete once the stream has been synchronised.  When
 * h_y is pinned, mapped host memory the kernel writes it directly, otherwise a copy
 * is enqueued behind the kernel.  (Q4Q8Linear::Forward, q4q8_linear.cpp:315-389, is
 * synchronous; a caller that issues a whole decode pass synchronises once.) */
int garnet_b200_w4a16_run_host_async(garnet_b200_w4a16_t h, const void* h_x, void* h_y, int m, void* stream);
/* A prepared list of host-buffer calls (a whole decode pass, say): linear i reads
 * h_xs[i] ([ms[i], K_i] bf16) and writes h_ys[i].  `batch_run` copies every distinct
 * input buffer to the device once, launches the linears back to back (programmatic
 * dependent launches), and writes all outputs to their host buffers with one kernel
 * (pinned, mapped buffers) or one copy each (pageable buffers); the outputs are
 * complete once `stream` has been synchronised.  When every call has the same batch of
 * at most 16 rows the linears run as one garnet_b200_w4a16_list launch, which writes
 * pinned, mapped output buffers itself while the pass runs.  Every h_xs[i]
 * and h_ys[i] must stay allocated, with unchanged pinning, until batch_destroy: the
 * device aliases of pinned outputs are taken at create time.  The reference's CPU backend calls
 * Q4Q8Linear::Forward once per operator (q4q8_linear.cpp:315-389); this is the same
 * list of calls handed over at once.  create/destroy allocate and free device memory;
 * run does not. */
typedef struct garnet_b200_w4a16_batch_s* garnet_b200_w4a16_batch_t;
int garnet_b200_w4a16_batch_create(const garnet_b200_w4a16_t* handles, const void* const* h_xs, void* const* h_ys,
                                   const int* ms, int count, garnet_b200_w4a16_batch_t* out);
int garnet_b200_w4a16_batch_run(garnet_b200_w4a16_batch_t batch, void* stream);
void garnet_b200_w4a16_batch_destroy(garnet_b200_w4a16_batch_t batch);

/* Writes the dequantised weights q*s as fp32 [n_local, k], reading the packed
 * tiles with the same device decode the GEMM kernels use (bit-exactness check;
 * cf. TestGptOssMxfp4Decode, plugins/gpt_oss/include/gpt_oss_kernels.h:65). */
int garnet_b200_w4a16_dequant(garnet_b200_w4a16_t h, float* d_out, void* stream);

/* Non-zero when a bounded device-side wait of this handle's kernels gave up
 * (read from mapped host memory; meaningful after the stream has been
 * synchronised).  The reference reports such faults through a fault word as
 * well (plugins/gpt_oss/cuda/tp_peer_owner.cuh:40-46,308-315). */
int garnet_b200_w4a16_fault(garnet_b200_w4a16_t h);

void garnet_b200_w4a16_destroy(garnet_b200_w4a16_t h);

/* ---- checkpoints and the packed-constant cache (host only) ---------------------
 * The reference reads weights through SafeTensorsIndex (src/model/safetensors_index.h:42-60:
 * a single .safetensors file, a Hugging Face model.safetensors.index.json, or a directory
 * holding either; tensors are views into memory-mapped files), quantizes Qwen linears with
 * QuantizeSymmetricINT4 (src/model/weight_quantization.cpp:188-270) and names the packed
 * constants it derives so that a stripped engine can regenerate them
 * (plugins/gpt_oss/include/gpt_oss_marlin_pack.h:29-44). */
typedef struct garnet_b200_safetensors* garnet_b200_safetensors_t;
int garnet_b200_safetensors_open(const char* path, garnet_b200_safetensors_t* out);
int garnet_b200_safetensors_count(garnet_b200_safetensors_t st);
/* One tensor, by `name` or (name == NULL) by `index` in file order: its name, dtype string
 * ("BF16", "U8", ...), rank, shape (up to 8 extents), a pointer into the mapped file (valid
 * until close) and its byte count.  Any output pointer may be NULL. */
int garnet_b200_safetensors_entry(garnet_b200_safetensors_t st, int index, const char* name, const char** name_out,
                                  const char** dtype, int* rank, long long* shape8, const void** data, size_t* bytes);
void garnet_b200_safetensors_close(garnet_b200_safetensors_t st);
/* Writes `count` tensors as one .safetensors file (data 256-byte aligned in the file). */
int garnet_b200_safetensors_write(const char* path, const char* const* names, const char* const* dtypes, const int* ranks,
                                  const long long* const* shapes, const void* const* datas, const size_t* bytes, int count);

/* QuantizeSymmetricINT4 on the host: w [n, k] of fp32 / fp16 / bf16 -> canonical nibbles and
 * fp16 (the reference's artifact) or bf16 scales; the same bits as garnet_b200_int4_quantize
 * writes on the device.  max_abs_error may be NULL. */
int garnet_b200_int4_quantize_host(const void* w, int w_dtype, int n, int k, int group, int scale_dtype, uint8_t* nibbles,
                                   uint16_t* scales, double* max_abs_error);

/* Names of derived constants: kind 0 = packed int4 linear ("__garnet_b200_w4a16_v1_g<a>_s<b>__:" +
 * source; a = group, b = scale dtype), kind 1 / 2 = MoE projection in the streaming / block
 * layout ("__garnet_b200_mxs|mxb_v1_u<a>_t<b>of<c>__:" + source; a = 0 gate_up, 1 down;
 * b of c = the intermediate-axis part, 0 of 1 when unsplit).  `parse` is the inverse. */
int garnet_b200_packed_tensor_name(const char* source, int kind, int a, int b, int c, char* out, size_t out_bytes);
int garnet_b200_packed_tensor_name_parse(const char* name, int* kind, int* a, int* b, int* c, const char** source);

/* Builds the packed-constant cache of a checkpoint as one .safetensors file: every tensor
 * that garnet_b200_is_int4_linear_weight accepts is quantized and packed
 * (garnet_b200_w4a16_create_prepacked takes the bytes as they are), every gpt-oss expert pair
 * <prefix>.mlp.mlp1_weight.{blocks,scales} / mlp2_weight.{blocks,scales}
 * (xModel/gpt_oss/120b/gpt_oss_llm.py:110-115) is packed in the layouts `moe_layouts` asks for
 * (0 both; for tp_world > 1 this rank's part of the intermediate axis), all under their derived
 * names; every other tensor is copied as it is.  One tensor at a time is held in memory. */
int garnet_b200_checkpoint_build_cache(garnet_b200_safetensors_t st, const char* out_path, int group, int scale_dtype,
                                       int moe_layouts, int tp_rank, int tp_world);

/* ---- the rest of a Qwen3 decode step ------------------------------------------
 * What sits between the int4 linears of a decoder layer and is not folded into a
 * garnet_b200_w4a16_list: attention of one new token per sequence over the paged bf16 KV
 * cache, the embedding row and the greedy token.  The reference runs these as separate
 * engines and kernels: the packed q/k/v lowering with per-head q/k RMS norm and rotate-half
 * RoPE (src/backends/tensorrt/trt_builder.cpp:7565-7726, :1815-1870), the cache append and
 * the split decode attention over page tables (src/cuda/text_kv_attention_kernel.cu:640-840)
 * and the greedy sampler (src/cuda/logits_sampler_kernel.cu). */
typedef struct garnet_b200_attention_options {
    int abi;                /* GARNET_B200_ABI */
    int struct_size;        /* sizeof(garnet_b200_attention_options) */
    int q_heads;            /* 16 for Qwen3-1.7B */
    int kv_heads;           /* 8; q head h reads kv head h / (q_heads / kv_heads) */
    int head_dim;           /* 128 (the only supported value) */
    int page_size;          /* positions per cache page (16 in the reference) */
    int max_logical_pages;  /* columns of the page table */
    int max_context;        /* largest context a call may see (sizes the grid and the workspace) */
    int rope_positions;     /* rows of the cos / sin tables */
    float norm_eps;         /* of the q / k head norms */
} garnet_b200_attention_options;

/* Workspace bytes for `batch` sequences.  The caller zero-fills the workspace once
 * (cudaMemset) before the first call; the kernel leaves its counters zero. */
int garnet_b200_attention_decode_workspace(const garnet_b200_attention_options* options, int batch, size_t* bytes);

/* d_qkv [batch, (q_heads + 2 kv_heads) * 128] bf16: the output row q | k | v of the packed
 * q/k/v linear.  Per sequence b with slot = d_positions[b] (its context is slots 0 .. slot):
 *   q_h  = rope(bf16(rmsnorm(q_h) * q_norm_weight), slot) for every q head, k likewise with
 *          k_norm_weight; rope uses rows `slot` of d_rope_cos / d_rope_sin (fp32 [rope_positions, 64],
 *          rotate-half: out[d] = x[d] cos[d] - x[d+64] sin[d], out[d+64] = x[d+64] cos[d] + x[d] sin[d]);
 *   k, v are written to the cache at ((page_table[b][slot / page_size] * page_size + slot % page_size)
 *          * kv_heads + kv_head) * 128 (the reference's layout, text_kv_attention_kernel.cu:668-673);
 *   out[b, h*128 ..] = softmax(q_h . K^T / sqrt(128)) V over the context, fp32 arithmetic, bf16 result.
 * flags bit 0: programmatic dependent launch.  No allocation, no synchronisation. */
int garnet_b200_attention_decode(const garnet_b200_attention_options* options, const void* d_qkv, const void* d_q_norm_weight,
                                 const void* d_k_norm_weight, const float* d_rope_cos, const float* d_rope_sin, void* d_key_pages,
                                 void* d_value_pages, const int* d_page_tables, const int* d_positions, void* d_out,
                                 void* d_workspace, size_t workspace_bytes, int batch, unsigned flags, void* stream);

/* out[b, :] = table[ids[b], :] (bf16 [vocab, hidden]; ids outside the table are clamped). */
int garnet_b200_embedding_gather(const void* d_table, const int* d_ids, void* d_out, int batch, int hidden, int vocab,
                                 unsigned flags, void* stream);

/* out[b] = index of the largest of logits[b, :vocab] (bf16), the lowest index among equals. */
int garnet_b200_argmax_bf16(const void* d_logits, int* d_out, int batch, int vocab, unsigned flags, void* stream);

/* ---- the rest of a gpt-oss decoder layer -----------------------------------------
 * The operators around the MoE that the reference's plugin also carries (GptOssOptions kinds 0, 1,
 * 5, 6, 7; plugins/gpt_oss/include/gpt_oss_kernels.h:8-46): RunGptOssRmsNorm, RunGptOssRope (YaRN),
 * RunGptOssAttention (paged bf16 KV cache, learned sinks, sliding window), RunGptOssDecodeGemv and
 * RunGptOssVocabTop1.  x and y are the reference's fp32 carrier (fp32 tensors holding bf16 values)
 * unless stated. */
typedef struct garnet_b200_gpt_oss_options {
    int abi;               /* GARNET_B200_ABI */
    int struct_size;       /* sizeof(garnet_b200_gpt_oss_options) */
    int q_heads, kv_heads, head_dim;      /* gpt-oss-120b: 64, 8, 64 */
    int layer;             /* selects the layer's slab of the KV cache */
    int page_size;         /* positions per cache page (16) */
    int window;            /* sliding window in positions, 0 = full attention */
    int prefill;           /* 1: row t attends positions up to starts[b] + t; 0: up to lengths[b] */
    float theta, factor, initial_context, beta_fast, beta_slow;   /* YaRN: 150000, 32, 4096, 32, 1 */
} garnet_b200_gpt_oss_options;

/* y = bf((bf(x) * rsqrt(mean(bf(x)^2) + epsilon)) * weight), rows of `hidden` (RunGptOssRmsNorm). */
int garnet_b200_gpt_oss_rms_norm(const float* d_x, const float* d_weight, float* d_y, int rows, int hidden, float epsilon,
                                 void* stream);
/* YaRN rotary embedding of the q and k heads of packed rows [tokens, (q + 2 kv) * d]; the v part
 * is copied (RunGptOssRope, gpt_oss_kernels.cu:78-99).  d_positions: int64 [tokens]. */
int garnet_b200_gpt_oss_rope(const garnet_b200_gpt_oss_options* options, const float* d_x, const long long* d_positions, float* d_y,
                             int tokens, void* stream);
/* in[0..7] = qkv f32 [batch * tokens, (q + 2 kv) * d] (rotated), key cache, value cache (bf16
 * [layers][physical pages][page size][kv heads][d]), page table int32 [batch, logical pages],
 * lengths int32 [batch], starts int32 [batch], active int32 [batch], sinks f32 [q heads]: appends the
 * rows' k and v at positions starts[b] + t, then y[row, head] = softmax over the visible window, with
 * the head's sink in the denominator only (RunGptOssAttention, gpt_oss_kernels.cu:1012-1210).
 * The workspace (zero-filled once by the caller) is needed at decode (tokens == 1, prefill == 0). */
int garnet_b200_gpt_oss_attention_workspace(const garnet_b200_gpt_oss_options* options, int batch, int logical_pages, size_t* bytes);
int garnet_b200_gpt_oss_attention(const garnet_b200_gpt_oss_options* options, const void* const* in, float* d_y, void* d_workspace,
                                  size_t workspace_bytes, int batch, int tokens, int logical_pages, int physical_pages, void* stream);
/* pairs[row] = (largest logit, float(rank * width + its index)), the lowest index among equals
 * (RunGptOssVocabTop1: the 8-byte message of the sharded vocabulary). */
int garnet_b200_gpt_oss_vocab_top1(const float* d_logits, float* d_pairs, int rows, int width, int rank, void* stream);
/* y[row] = bf16(sum_c W[row', column_offset + c] * x[c]) for bf16 x, W, y; with q_heads > 0 row' walks
 * this rank's half of the q, k and v rows of a packed q/k/v weight (RunGptOssDecodeGemv,
 * plugins/gpt_oss/cuda/gpt_oss_gemv.cu:7-60). */
int garnet_b200_gpt_oss_decode_gemv(const void* d_x, const void* d_weight, void* d_y, int rows, int columns, int weight_stride,
                                    int column_offset, int q_heads, int kv_heads, int head_dim, int rank, void* stream);

/* ---- gpt-oss MXFP4 mixture of experts (`gpt_oss_moe_mxfp4`) -------------------
 * Replaces the free functions below the TensorRT plugin:
 *   size_t GptOssMoeWorkspace(int tokens, const GptOssOptions&) and
 *   cudaError_t RunGptOssMoe(const void* const* in, float* y, void* workspace, int tokens,
 *                            const GptOssOptions&, cudaStream_t)
 * (plugins/gpt_oss/include/gpt_oss_kernels.h:41-43), and the stateful
 * GptOssMarlin{ctor, Workspace, Run} (plugins/gpt_oss/include/gpt_oss_marlin.h:17-30).
 *
 * Options mirror the GptOssOptions fields the MoE uses
 * (plugins/gpt_oss/include/gpt_oss_kernels.h:8-20): hidden, intermediate, experts,
 * topK, prefill, limit, tpRank (-> ep_rank with ep_world = 2, ep_interleaved = 1),
 * expertWeightsSharded.  `abi` and `struct_size` version the struct the way the
 * reference versions its module bridge (src/model/operator_module_bridge.h:6-14). */
typedef struct garnet_b200_moe_options {
    int abi;                    /* GARNET_B200_ABI */
    int struct_size;            /* sizeof(garnet_b200_moe_options) */
    int hidden;
    int intermediate;
    int experts;
    int top_k;
    int prefill;                /* informational; the kernel choice follows the token count */
    int ep_rank;                /* expert-parallel rank; ignored when ep_world <= 1 */
    int ep_world;               /* 0 or 1 = unsharded */
    int ep_interleaved;         /* 1: expert e belongs to rank e % ep_world (reference rule);
                                   0: contiguous blocks of experts / ep_world */
    int expert_weights_sharded; /* expert tensors (and biases) hold only this rank's experts */
    int io_dtype;               /* GARNET_B200_FP32 (reference carrier: fp32 holding bf16 values) or GARNET_B200_BF16 */
    float limit;                /* swiglu clamp, 7 for gpt-oss */
    /* Fields below were added after the first version of the struct: a caller that
     * passes the earlier struct_size (up to and including `limit`) gets zeros here. */
    int layouts;                /* which packed copies of the experts the handle holds:
                                   0 both (any token count at full speed), GARNET_B200_MOE_LAYOUT_STREAM
                                   (decode: few rows per expert), GARNET_B200_MOE_LAYOUT_BLOCK
                                   (prefill: block-scaled tensor-core tiles).  With one copy the
                                   handle holds the experts once and every token count runs on it. */
    int tp_rank;                /* intermediate-axis split (the reference's "inner" 2-way tensor */
    int tp_world;               /* parallelism, gpt_oss_weight_shard.h:9-11): rank r computes
                                   intermediate channels [r I/world, (r+1) I/world): gate/up row pairs
                                   and down-projection K groups; the down bias is added on rank 0
                                   only; the output is this rank's unrounded partial sum, to be
                                   all-reduced.  0 or 1 = not split.  `intermediate` is always the
                                   full width. */
    int tp_weights_sharded;     /* the expert tensors and the gate/up bias already hold only this
                                   rank's part (GatherGptOssIntermediateShard modes 1 and 2) */
} garnet_b200_moe_options;

enum { GARNET_B200_MOE_LAYOUT_BOTH = 0, GARNET_B200_MOE_LAYOUT_STREAM = 1, GARNET_B200_MOE_LAYOUT_BLOCK = 2 };

typedef struct garnet_b200_moe* garnet_b200_moe_t;

/* Caller-provided workspace size for `tokens` tokens.  GptOssMoeWorkspace
 * (gpt_oss_kernels.h:41). */
int garnet_b200_moe_workspace(const garnet_b200_moe_options* options, int tokens, size_t* bytes);

/* Creates the operator.  `weights[0..7]` are operands in[1..8] of the reference
 * operand list (src/backends/tensorrt/gpt_oss_lowering.cpp:309-312), device
 * resident, original checkpoint layout: router W [E,H] f32, router b [E] f32,
 * gate_up blocks u8 [E,2I,H/32,16], gate_up scales u8 [E,2I,H/32], gate_up bias
 * [E,2I] f32, down blocks [E,H,I/32,16], down scales [E,H,I/32], down bias [E,H]
 * f32.  Expert blocks and scales are repacked into handle-owned memory (one
 * stream synchronise): in the layout of the streaming kernels (few rows per
 * expert) and as the blocks and scale atoms of the block-scaled tensor-core
 * kernels (many rows per expert) - both when options->layouts is 0, so that a
 * handle then holds about twice the size of the expert tensors, or only the one
 * that options->layouts names; router weights and biases are borrowed and must outlive the
 * handle (the router weight is also kept as three bf16 terms for the tensor-core
 * router).  GptOssMarlin constructor + first-run prepare
 * (plugins/gpt_oss/cuda/gpt_oss_marlin.cu:415-499). */
int garnet_b200_moe_create(const garnet_b200_moe_options* options, const void* const* weights, void* stream,
                           garnet_b200_moe_t* out);

/* y[tokens, hidden] = MoE(x[tokens, hidden]); x and y are of io_dtype and 16-byte
 * aligned (as are the row and value buffers of every entry point below; the
 * kernels use 16-byte vector accesses, and a misaligned pointer is rejected with
 * INVALID_VALUE before anything is launched).  No allocation, no synchronisation.  RunGptOssMoe / GptOssMarlin::Run
 * (gpt_oss_kernels.h:42-43, gpt_oss_marlin.h:28-29).  With ep_world > 1 the output
 * is this rank's unrounded partial sum (gpt_oss_kernels.cu:810). */
int garnet_b200_moe_run(garnet_b200_moe_t h, const void* d_x, void* d_y, void* d_workspace, size_t workspace_bytes,
                        int tokens, void* stream);

/* Same computation as garnet_b200_moe_run for callers that have no workspace to
 * give and may not create one.  (No counterpart in the reference, whose callers
 * always receive a workspace from the engine that owns the plugin.)  It is meant
 * for hosts that drive this library directly from a latency-critical decode loop
 * in which device allocation is off limits: cudaMalloc and cudaFree serialise
 * with all work on the device, and in deployments where another runtime has
 * already reserved the GPU's memory they simply fail.  The scratch is a 8 MiB
 * array built into the library image (held by every GPU that loads the library,
 * until the process exits); this call allocates and frees nothing, on the host
 * side of CUDA or through any library.
 *   - Limit: the layer's workspace for `tokens` must fit in 8 MiB - 111 tokens for
 *     the gpt-oss-120b layer (hidden = intermediate = 2880, 128 experts, top-4).
 *     Larger requests are rejected with INVALID_VALUE and a message that names the
 *     largest token count that fits.
 *   - The array's device address is looked up once per device by
 *     garnet_b200_moe_create (with that device current), never by this call; create
 *     the handle before starting any stream capture on that device.  The call must
 *     be made with the device current on which the handle was created; any other
 *     device is rejected with INVALID_VALUE.
 *   - All calls on a device share the one array, and it keeps the previous call's
 *     contents.  Nothing needs clearing between calls, but two calls whose kernels
 *     overlap on the GPU (different streams, or different handles at once) race on
 *     it: serialise them, or use garnet_b200_moe_run with separate workspaces. */
int garnet_b200_moe_run_static(garnet_b200_moe_t h, const void* d_x, void* d_y, int tokens, void* stream);

/* ---- expert-parallel building blocks --------------------------------------------
 * The reference shards experts two ways with replicated tokens and an all-reduce
 * of partial sums (expert % 2 == rank, plugins/gpt_oss/cuda/gpt_oss_kernels.cu:771,
 * :818; xModel/gpt_oss/120b/gpt_oss_llm.py:119-123) - garnet_b200_moe_run with
 * ep_world > 1 reproduces that.  For wider expert parallelism over NVLink the
 * tokens are instead exchanged: each rank routes its own tokens
 * (garnet_b200_moe_route), rows travel to the rank that owns their expert, that
 * rank runs the experts on the rows it received (garnet_b200_moe_run_rows), the
 * per-row values travel back and the source rank applies the router weights in
 * router order (garnet_b200_moe_combine, gpt_oss_kernels.cu:907-921).  The
 * exchange itself is the caller's (NCCL all-to-all in garnet_b200/dist.py). */

/* Workspace bytes of garnet_b200_moe_run_rows for `rows` rows. */
int garnet_b200_moe_rows_workspace(const garnet_b200_moe_options* options, int rows, size_t* bytes);

/* d_vals[r, :] (fp32, bf16-valued) = bf(bf(h_r . w_down[e]) + bd[e]) with
 * h_r = SwiGLU(d_rows[r, :] . w_gate_up[e] + b) and e = d_row_expert[r] (global
 * expert id; must be one of this handle's experts, other rows are skipped).
 * d_rows is [rows, hidden] of io_dtype. */
int garnet_b200_moe_run_rows(garnet_b200_moe_t h, const void* d_rows, const int* d_row_expert, int rows,
                             float* d_vals, void* d_workspace, size_t workspace_bytes, void* stream);

/* The two halves of garnet_b200_moe_run_rows on their own, as the reference runs
 * them (gate/up GEMM + activation, then the down GEMM:
 * plugins/gpt_oss/cuda/gpt_oss_marlin.cu:632-644):
 *   stage 1: d_hidden[r, :] (fp32 [rows, intermediate], bf16-valued) =
 *            SwiGLU(d_rows[r, :] . w_gate_up[e] + b); d_vals is not used;
 *   stage 2: d_vals[r, :] = bf(bf(d_hidden[r, :] . w_down[e]) + bd[e]); d_rows is not used.
 * Same workspace as garnet_b200_moe_run_rows.  Lets each projection be checked
 * against the reference arithmetic by itself. */
int garnet_b200_moe_run_rows_stage(garnet_b200_moe_t h, int stage, const void* d_rows, const int* d_row_expert, int rows,
                                   float* d_hidden, float* d_vals, void* d_workspace, size_t workspace_bytes, void* stream);

/* y[t, :] = bf(sum_j d_vals[t * top_k + j, :] * d_probs[t, j]), j in router order
 * (combineExperts, gpt_oss_kernels.cu:907-921). */
int garnet_b200_moe_combine(garnet_b200_moe_t h, const float* d_vals, const float* d_probs, void* d_y, int tokens,
                            void* stream);

/* Router only: bf16-rounded logits [tokens, experts], top-k expert ids
 * [tokens, top_k] and bf16-rounded probabilities.  RunGptOssMoeRoute
 * (gpt_oss_kernels.h:54-56). */
int garnet_b200_moe_route(garnet_b200_moe_t h, const void* d_x, int* d_selected, float* d_probs, float* d_logits,
                          int tokens, void* stream);

/* The router exactly as garnet_b200_moe_run evaluates it for the same token count (many
 * tokens: scores on the tensor cores, the fp32 router weight as three bf16 terms with
 * fp32 accumulation; garnet_b200_moe_route always uses the fp32 pipe, and its logits
 * can differ from these in the last bf16 step).  The expert-parallel flow routes with
 * this entry point.  Workspace size from garnet_b200_moe_route_workspace. */
int garnet_b200_moe_route_workspace(const garnet_b200_moe_options* options, int tokens, size_t* bytes);
int garnet_b200_moe_route_ws(garnet_b200_moe_t h, const void* d_x, int* d_selected, float* d_probs, float* d_logits,
                             int tokens, void* d_workspace, size_t workspace_bytes, void* stream);

/* Decodes rows x 32 MXFP4 values (16 bytes and one e8m0 byte per row) to fp32.
 * TestGptOssMxfp4Decode (gpt_oss_kernels.h:65). */
int garnet_b200_mxfp4_decode(const uint8_t* d_blocks, const uint8_t* d_scales, float* d_out, int rows, void* stream);

/* Writes one stored expert matrix (which = 0: gate_up [2I,H], 1: down [H,I]) as
 * fp32 in the original row order, decoded from the packed tiles of the streaming
 * kernels; which = 2, 3: the same two matrices decoded from the second copy, the
 * blocks and scale atoms that the block-scaled tensor-core kernels read
 * (cf. the reference's packed-weight check, test2026/gpt_oss/marlin_weight_pack.cpp:54-78). */
int garnet_b200_moe_dequant(garnet_b200_moe_t h, int which, int stored_expert, float* d_out, void* stream);

/* ---- packed expert constants (host packer, borrowed prepacked form) ---------
 * The reference lets an engine hold the experts as derived constants that were packed
 * on the host, and hands them to the operator with marlinPrepacked = true
 * (PackGptOssMarlinWeight, plugins/gpt_oss/include/gpt_oss_marlin_pack.h:74-193;
 * gpt_oss_kernels.h:18; the test that host and device bytes agree:
 * test2026/gpt_oss/marlin_weight_pack.cpp:33-111, kernel_parity.cpp:576-586).
 *
 * A packed blob holds one projection (`which` = 0 gate_up, 1 down) of `experts`
 * experts in one layout: GARNET_B200_MOE_LAYOUT_STREAM = strips of 16 rows in 544-byte
 * chunks (codes + scale bytes), GARNET_B200_MOE_LAYOUT_BLOCK = 15 KiB blocks of 240 rows
 * x 128 columns followed by all their scale atoms.  With tp_world > 1 in `options` the
 * sizes are those of the rank's part (intermediate / tp_world). */
int garnet_b200_moe_packed_bytes(const garnet_b200_moe_options* options, int which, int layout, int experts, size_t* bytes);

/* Packs `experts` experts of one projection on the host: blocks [experts, rows, K/32, 16]
 * and scales [experts, rows, K/32] in the checkpoint layout (rows = 2I and K = H for
 * gate_up, rows = H and K = I for down; rank-local I when tp_world > 1), into `out`
 * (garnet_b200_moe_packed_bytes bytes).  Byte for byte what garnet_b200_moe_create
 * builds on the device.  Uses up to 16 host threads, as the reference's packer does. */
int garnet_b200_moe_pack_host(const garnet_b200_moe_options* options, int which, int layout, const uint8_t* blocks,
                              const uint8_t* scales, int experts, uint8_t* out);

/* The handle's own packed blob of a projection in a layout (device pointer and size),
 * or NOT_SUPPORTED when the handle does not hold that layout. */
int garnet_b200_moe_packed_view(garnet_b200_moe_t h, int which, int layout, const void** d_blob, size_t* bytes);

/* Creates the operator over packed blobs that the caller owns and keeps alive (device
 * memory, 256-byte aligned): nothing is repacked and the experts are not copied.
 * small[0..3] = router W [E,H] f32, router b [E] f32, gate_up bias [E_local, 2 I_local] f32,
 * down bias [E_local, H] f32; packed[0..3] = gate_up stream, down stream, gate_up block,
 * down block - those that options->layouts asks for (both pairs when it is 0), each
 * holding this rank's experts only.  GptOssMarlin with marlinPrepacked
 * (plugins/gpt_oss/cuda/gpt_oss_marlin.cu:427-433,487-499). */
int garnet_b200_moe_create_prepacked(const garnet_b200_moe_options* options, const void* const* small,
                                     const void* const* packed, void* stream, garnet_b200_moe_t* out);

/* Rank-local part of a checkpoint tensor for the intermediate-axis split, on the host:
 * GatherGptOssIntermediateShard (src/backends/tensorrt/gpt_oss_weight_shard.h:25-60)
 * for any world size.  mode 1: the rank's slice of axis 1 (gate_up blocks, scales, bias);
 * mode 2: of axis 2 (down blocks, scales); mode 3: the whole tensor on rank 0, zeros on the
 * others (down bias).  `shape` has `rank_dims` extents (2..4); `out` takes bytes / world
 * bytes (modes 1, 2) or bytes (mode 3). */
int garnet_b200_moe_gather_intermediate_shard(const void* source, size_t bytes, const long long* shape, int rank_dims,
                                              size_t element_bytes, int rank, int world, int mode, void* out);

/* The activation format of the block-scaled tensor-core path, on its own: every
 * 32-block of a bf16 row [rows, k] becomes two e4m3 rows (d_hi, d_lo: [rows, k] bytes)
 * that share one e8m0 scale byte (d_scales: [rows, k/32]): x = (hi + lo) * 2^(scale-127),
 * exactly for elements within 2^-9 of the block's largest magnitude and to 2^-17 of it
 * otherwise.  A block that holds an infinity or a NaN gets scale byte 255 (NaN).  For
 * checks of the split; the reference keeps activations in bf16
 * (plugins/gpt_oss/cuda/gpt_oss_marlin.cu:586-590). */
int garnet_b200_mx_split_rows(const void* d_x_bf16, int rows, int k, uint8_t* d_hi, uint8_t* d_lo, uint8_t* d_scales,
                              void* stream);

/* Non-zero when a bounded device-side wait gave up (see garnet_b200_w4a16_fault). */
int garnet_b200_moe_fault(garnet_b200_moe_t h);

/* ---- collectives over NVLink (one node, up to 8 ranks) ---------------------------
 * Replace the reference's two-rank collectives GptOssTpAllReduce, GptOssTpAllReduceBf16
 * and GptOssTpAllGather (plugins/gpt_oss/cuda/tp_collective.cpp:77-148) and its
 * peer-memory all-reduce with bounded waits and a fault word
 * (plugins/gpt_oss/cuda/tp_peer_owner.cuh:30-106).  Every rank (one host thread or
 * process per GPU, that device current: tp_collective.cpp:82-85) owns an arena of
 * device memory which its peers map through CUDA IPC; contributions and flags are
 * stored directly into the destination GPU's own memory, every wait polls local
 * memory only and gives up after a time limit (status: garnet_b200_comm_fault; the
 * kernel returns, the context stays usable).  No host synchronisation on the data
 * path.  Set-up: create -> export a blob -> exchange the blobs of all ranks over any
 * host channel -> connect.  Objects carved from an arena (channels, the
 * expert-parallel exchange below) must be created in the same order on every rank. */
typedef struct garnet_b200_comm* garnet_b200_comm_t;
typedef struct garnet_b200_channel* garnet_b200_channel_t;
#define GARNET_B200_COMM_BLOB_BYTES 128
int garnet_b200_comm_create(int rank, int world, size_t arena_bytes, garnet_b200_comm_t* out);
int garnet_b200_comm_export(garnet_b200_comm_t comm, void* blob, size_t blob_bytes);
/* `blobs`: world consecutive blobs in rank order (this rank's own is ignored). */
int garnet_b200_comm_connect(garnet_b200_comm_t comm, const void* blobs);
int garnet_b200_comm_fault(garnet_b200_comm_t comm);
void garnet_b200_comm_destroy(garnet_b200_comm_t comm);

/* A channel carries collectives of up to slot_bytes per rank (two regions of
 * world x slot_bytes in the arena, alternating from call to call). */
int garnet_b200_comm_channel_create(garnet_b200_comm_t comm, size_t slot_bytes, garnet_b200_channel_t* out);
void garnet_b200_comm_channel_destroy(garnet_b200_channel_t channel);

/* d_dst[r] (r = 0..world-1, `bytes` each, contiguous) = d_src of rank r.  One kernel per
 * rank; bytes a multiple of 16.  GptOssTpAllGather (tp_collective.cpp:124-148); the
 * N-sharded lm_head gathers its logits with it. */
int garnet_b200_comm_all_gather(garnet_b200_channel_t channel, const void* d_src, size_t bytes, void* d_dst, void* stream);

/* d_dst[i] = sum over ranks of d_src[i], added in rank order on every rank (so all
 * ranks hold the same bits).  wire_dtype GARNET_B200_FP32: GptOssTpAllReduce
 * (tp_collective.cpp:77-98).  GARNET_B200_BF16: contributions travel as bf16 and the
 * fp32 sum is rounded to bf16, which for two ranks is exactly bf16(a + b):
 * GptOssTpAllReduceBf16 (tp_collective.cpp:100-122, tp_peer_math.cuh:10-14). */
int garnet_b200_comm_all_reduce(garnet_b200_channel_t channel, const float* d_src, float* d_dst, size_t count,
                                int wire_dtype, void* stream);

/* The same sum for bf16 tensors: d_src and d_dst hold `count` bf16 values; the contributions
 * travel as they are, are added in fp32 in rank order and rounded once - for two ranks
 * exactly the reference's wire rule bf16(a + b) (plugins/gpt_oss/cuda/tp_peer_math.cuh:10-14).
 * This is the reduction behind K-sharded ("row"-parallel) linears. */
int garnet_b200_comm_all_reduce_bf16(garnet_b200_channel_t channel, const void* d_src, void* d_dst, size_t count, void* stream);

/* ---- expert-parallel MoE with the exchange on the device ------------------------------
 * Tokens are split over the ranks, experts live in contiguous blocks of experts/world
 * (create the operator with ep_rank/ep_world of the communicator, ep_interleaved = 0,
 * io_dtype bf16; rank-local expert tensors with expert_weights_sharded = 1).  One call
 * routes this rank's tokens, stores every routed row into the receive buffer of the GPU
 * that owns its expert (plain peer stores; fixed-capacity regions per source, so no
 * count is needed before the data moves), runs the experts on what this rank
 * received, stores the per-row values back the same way (as bf16: exact) and combines in
 * router order: the output equals the single-GPU operator's.  No host synchronisation,
 * no library collective; every wait is bounded (garnet_b200_comm_fault).  All ranks
 * call it once per step.  The reference's form is two ranks with replicated tokens and
 * an all-reduce (plugins/gpt_oss/cuda/gpt_oss_kernels.cu:771,818), which
 * garnet_b200_moe_run with ep_world > 1 plus garnet_b200_comm_all_reduce reproduces. */
typedef struct garnet_b200_moe_ep* garnet_b200_moe_ep_t;
/* Arena bytes one exchange takes (add the channels' needs when sizing garnet_b200_comm_create). */
int garnet_b200_moe_ep_arena_bytes(const garnet_b200_moe_options* options, int world, int tokens_local_max, size_t* bytes);
int garnet_b200_moe_ep_create(garnet_b200_moe_t moe, garnet_b200_comm_t comm, int tokens_local_max, garnet_b200_moe_ep_t* out);
int garnet_b200_moe_ep_run(garnet_b200_moe_ep_t ep, const void* d_x, void* d_y, int tokens_local, void* stream);
/* Rows this rank's experts processed in the last completed call (read after a stream synchronise). */
int garnet_b200_moe_ep_rows_received(garnet_b200_moe_ep_t ep);
void garnet_b200_moe_ep_destroy(garnet_b200_moe_ep_t ep);
/* The exchange's placement rule on the host: send_idx[s] = position of routed row s
 * (expert selected[s], owner selected[s] / experts_per_rank) among the rows this rank
 * sends to that owner, in slot order; dest_count[d] = rows bound for rank d. */
int garnet_b200_moe_ep_plan_host(const int* selected, int slots, int experts_per_rank, int world, int* send_idx, int* dest_count);

/* Launches a wait on a flag that no peer ever writes, with the given limit (1..2000
 * ms), synchronises and returns DEVICE_FAULT: how every wait of the collectives ends
 * when a peer never shows up. */
int garnet_b200_comm_selftest_wait(garnet_b200_comm_t comm, int limit_ms, void* stream);

void garnet_b200_moe_destroy(garnet_b200_moe_t h);

#ifdef __cplusplus
}
#endif
#endif /* GARNET_B200_H */
