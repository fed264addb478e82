/* mxb200: a B200-native (sm_100a) MXFP8 Linear engine behind a C ABI.
 *
 * Drop-in for the torch-free kernel seam of nanochat-cpp's --fp8-recipe=mxfp8 / --gemm backend
 * (namespace nanochat::kernels). Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, a cudaStream_t), launches asynchronously on that stream against the current device and
 * returns an mxb200_status. Nothing here allocates device memory unless its comment says so; outputs,
 * scale buffers and the optional split-K workspace belong to the caller. There is no CPU fallback: on a
 * machine without an sm_100 GPU the calls fail with MXB200_ERR_DEVICE.
 *
 * Layout contract (src/nanochat/model/fp8/fp8_kernel.h:24-39, mx_kernel.cuh:29-44 in nanochat-cpp):
 *  - data: E4M3 bytes, row-major; one E8M0 scale byte per 32 consecutive values of a row, the smallest power
 *    of two with max|block| * 2^-e <= 448 (or the floor rule, see mxb200_scale_rule).
 *  - scales: cuBLAS's swizzled layout, 128 rows x 4 blocks per 512-byte tile, tiles row-major; the byte of
 *    (row r, block b) is ((r >> 7) * tiles + (b >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (b & 3).
 */
#ifndef MXB200_H_
#define MXB200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define MXB200_API __attribute__((visibility("default")))
#else
#define MXB200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mxb200_status {
  MXB200_OK = 0,
  MXB200_ERR_SHAPE = 1,      /* a dimension is not a multiple the kernel needs, or is not positive */
  MXB200_ERR_ALIGNMENT = 2,  /* a pointer or leading dimension is not 16-byte aligned */
  MXB200_ERR_NULL = 3,       /* a required pointer is null */
  MXB200_ERR_ARGUMENT = 4,   /* an enum or flag is out of range, or a combination is unsupported */
  MXB200_ERR_WORKSPACE = 5,  /* the workspace is missing or smaller than mxb200_gemm_workspace_bytes says */
  MXB200_ERR_DEVICE = 6,     /* no CUDA device, or the current device is not sm_100 */
  MXB200_ERR_DRIVER = 7,     /* the driver refused a tensor-map encode */
  MXB200_ERR_LAUNCH = 8,     /* the kernel launch itself failed (cudaGetLastError) */
  MXB200_ERR_WATCHDOG = 9    /* a bounded device-side wait ran out; see mxb200_device_status */
} mxb200_status;

/* Which power of two scales a block. REFERENCE is nanochat-cpp's rule, 2^ceil(log2(amax / 448)), which never
 * needs saturation (mx_kernel.cuh:29-34). OCP_FLOOR is 2^(floor(log2(amax)) - 8); values in (448, 512) times
 * the scale then saturate to +-448. */
typedef enum mxb200_scale_rule { MXB200_SCALE_REFERENCE = 0, MXB200_SCALE_OCP_FLOOR = 1 } mxb200_scale_rule;

/* Value transform applied while loading, before the block maximum (fp8_kernel.cu:44-50). */
typedef enum mxb200_prologue { MXB200_PROLOGUE_NONE = 0, MXB200_PROLOGUE_RELU_SQUARE = 1 } mxb200_prologue;

/* Where one layout of a quantized tensor goes. ABI-identical to nanochat::kernels::MxOut
 * (src/nanochat/model/fp8/fp8_kernel.h:28-33), so a sub-block of a larger buffer (merged q/k/v) is a view:
 * data + row0 * ld + col0, scale + ((row0 / 128) * scale_tiles + col0 / 128) * 512 (fp8.cpp:117-120). */
typedef struct mxb200_mx_out {
  void* data;          /* e4m3; null: this layout is not written */
  int64_t ld;          /* row stride of data, bytes */
  void* scale;         /* e8m0, at this view's first tile */
  int64_t scale_tiles; /* tiles per 128 rows in the whole scale buffer (its blocks per row / 4) */
} mxb200_mx_out;

/* Replaces nanochat::kernels::quantize_mx (src/nanochat/model/fp8/fp8_kernel.h:35-39; kernels
 * nanochat_mx_quantize_{bf16,f32,relu_square_bf16}, fp8_kernel.cu:197-205).
 * x: (rows, cols) contiguous bf16 (x_bf16 != 0) or fp32. out: x scaled along its rows; out_t: x's transpose
 * (cols, rows) scaled along its own rows. rows, cols % 128 == 0 (the callers' mx_fits, fp8.h:86-88);
 * x, data pointers and lds 16-byte aligned. prologue RELU_SQUARE quantizes bf16(relu(x)^2), bf16 x only.
 * Plain bf16 tensors of more than four tiles of 128 x 128 per SM run as persistent CTAs that draw their tiles from a
 * counter in the library's device image; at most 256 such launches may be in flight on a device at once (launches on
 * one stream never overlap; this bounds launches spread over many streams). */
MXB200_API int mxb200_quantize_mx(const void* x, int x_bf16, int64_t rows, int64_t cols, mxb200_mx_out out, mxb200_mx_out out_t,
                       int prologue, int scale_rule, void* stream);

/* One tensor of mxb200_quantize_mx_batch: the arguments of mxb200_quantize_mx that differ per tensor. */
typedef struct mxb200_quantize_job {
  const void* x;
  int64_t rows, cols;
  mxb200_mx_out out, out_t;
} mxb200_quantize_job;

/* mxb200_quantize_mx (no prologue) of n_jobs tensors of one input type in as few launches as possible (32 tensors
 * each), bit for bit what n_jobs separate calls give. It stands for the runs of quantize_mx calls the reference makes
 * on small tensors: the three parts of the merged q/k/v weight (src/nanochat/model/fp8/fp8.cpp:155-171) and a model's
 * weights after an optimizer step (Fp8WeightCache, fp8.cpp:516-536), where a launch per matrix of one or two waves of
 * tiles is bound by its own ramp-up and tail. jobs is read on the host during the call. */
MXB200_API int mxb200_quantize_mx_batch(const mxb200_quantize_job* jobs, int n_jobs, int x_bf16, int scale_rule,
                                        void* stream);

/* Replaces nanochat::kernels::quantize_mx_relu_square_bwd (fp8_kernel.h:41-43, fp8_kernel.cu:207-210):
 * quantizes dh = bf16(h > 0 ? g * 2h : 0) from bf16 g, h (rows, cols) without writing dh. */
MXB200_API int mxb200_quantize_mx_relu_square_bwd(const void* g, const void* h, int64_t rows, int64_t cols, mxb200_mx_out out,
                                       mxb200_mx_out out_t, int scale_rule, void* stream);

/* Loss pass of the chunked lm_head: replaces nanochat::kernels::softcap_ce with grad = false
 * (src/nanochat/model/ops/softcap_ce_kernel.h:13-22), the form the MX branch uses (ops/softcap_ce.cpp:66-71).
 * logits: (rows, ld) bf16, columns [0, padded) used, columns >= vocab ignored; padded, ld % 8 == 0. targets: (rows)
 * int64 on the device, < 0 = ignored. With capped = softcap * tanh(z / softcap): lse[row] = log sum exp(capped)
 * (unset for ignored rows), loss[row] = lse - capped[target] (0 for ignored rows). loss or lse may be null. */
MXB200_API int mxb200_softcap_ce_loss(const void* logits, int64_t rows, int64_t ld, const int64_t* targets, int vocab,
                                      int padded, float softcap, float* loss, float* lse, void* stream);

/* Replaces nanochat::kernels::softcap_ce_grad_mx (softcap_ce_kernel.h:24-29; kernel nanochat_softcap_ce_grad_mx,
 * softcap_ce_kernel.cu:118-176): the loss's gradient with respect to the logits, as the bf16 the reference's grad
 * kernel would write, g = bf16((softmax(capped) - onehot(target)) * (1 - tanh^2) * scale), MX-quantized in both
 * layouts without being written. scale = grad_scale[row * grad_scale_stride] (null: 1) / *num_valid (null: 1), both
 * on the device; rows with target < 0 and columns >= vocab give 0. rows, padded % 128 == 0. */
MXB200_API int mxb200_softcap_ce_grad_mx(const void* logits, int64_t rows, int64_t ld, const int64_t* targets,
                                         const float* lse, int vocab, int padded, float softcap,
                                         const float* grad_scale, int64_t grad_scale_stride, const int64_t* num_valid,
                                         mxb200_mx_out out, mxb200_mx_out out_t, int scale_rule, void* stream);

/* Arguments of mxb200_residual_norm_mx_fwd; the fields of nanochat::kernels::ResidualNormMxFwd and its base
 * ResidualNormFwd (src/nanochat/model/ops/residual_norm_kernel.h:17-41) in one flat struct. All tensors are
 * (rows, cols) contiguous bf16 unless noted, 16-byte aligned. */
typedef struct mxb200_residual_norm_mx {
  const void* x;    /* the residual stream */
  const void* r;    /* added to x first (the previous block's output); null: no add */
  const void* x0;   /* blended in with the layer's lambdas; null: no blend */
  const float* lr;  /* device fp32 scalars, required with x0 */
  const float* l0;
  void* s;          /* out, optional: bf16(x + r), kept for the lambdas' gradients when both r and x0 are given */
  void* res;        /* out: the new residual stream */
  void* n;          /* out, (rows, cols): only columns [0, n_cols) of the normalized rows are written, rounded up to
                       whole 8-column vectors (the value-embedding gate reads them); may be null when n_cols == 0 */
  float* rstd;      /* out: (rows) fp32 reciprocal RMS per row */
  int64_t rows;
  int32_t cols;
  float eps;
  mxb200_mx_out out;   /* MX of n: (rows, cols) scaled along rows */
  mxb200_mx_out out_t; /* MX of n^T: (cols, rows) */
  int32_t n_cols;
} mxb200_residual_norm_mx;

/* Replaces nanochat::kernels::residual_norm_mx_fwd (src/nanochat/model/ops/residual_norm_kernel.h:28-41, kernels
 * nanochat_residual_norm_mx_fwd_c*, residual_norm_kernel.cu:153-214): per row s = bf16(x + r),
 * res = bf16(bf16(lr * s) + bf16(l0 * x0)), n = bf16(res * rsqrt(mean(res^2) + eps)), and n leaves MX-quantized in
 * both layouts instead of being written, bit for bit what mxb200_quantize_mx of the bf16 n would give. It is the
 * producer of the quantized input of the QKV and MLP-fc GEMMs. rows, cols % 128 == 0, cols <= 2048. */
MXB200_API int mxb200_residual_norm_mx_fwd(const mxb200_residual_norm_mx* args, void* stream);

/* Replaces nanochat::kernels::cutlass_mx_gemm_bf16 (src/nanochat/model/fp8/mx_gemm_kernel.h:13-17).
 * d (M, N) bf16 row-major = a (M, K) . b (N, K)^T; a, b row-major e4m3 with their swizzled e8m0 scales along K;
 * fp32 accumulation, one round-to-nearest-even to bf16. M, N, K % 128 == 0, pointers 16-byte aligned.
 * resid (optional, (M, N) bf16): the fused residual add, d = bf16(float(bf16(acc)) + float(resid)), the two
 * roundings of the reference's separate add (src/nanochat/model/ops/residual_norm_kernel.cu:96-104).
 * resid may alias d. Needs no workspace. Launches on different streams of one device may overlap; at most 1024 GEMM
 * launches of this library may be in flight on a device at once (each holds one of 1024 scheduler slots in the
 * library's device image until its kernel exits; the same limit applies to concurrent replays of one CUDA graph,
 * whose launches keep the slot they were captured with). */
MXB200_API int mxb200_gemm_bf16(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d, const void* resid,
                     int64_t M, int64_t N, int64_t K, void* stream);

/* Replaces nanochat::kernels::cutlass_mx_gemm_f32 (mx_gemm_kernel.h:19-22): fp32 d (+)= alpha * a . b^T.
 * alpha: a device fp32 scalar or null (= 1); accumulate != 0: d += (beta 1), else d =. Needs no workspace
 * (one CTA owns each output tile for the whole of K). */
MXB200_API int mxb200_gemm_f32(const void* a, const void* a_scale, const void* b, const void* b_scale, float* d, int64_t M,
                    int64_t N, int64_t K, const float* alpha, int accumulate, void* stream);

/* Replaces nanochat::kernels::cutlass_mx_gemm_relu_square (src/nanochat/model/fp8/mx_gemm_kernel.h:24-27; used by the
 * MLP forward, fp8.cpp:279-284): h (M, N) bf16 = a . b^T as mxb200_gemm_bf16, and in the same epilogue the outputs
 * of mxb200_quantize_mx(h, RELU_SQUARE), bit for bit: q (M, N) e4m3 + q_scale, q_t (N, M) e4m3 + q_t_scale, each
 * a whole contiguous tensor with its own swizzled scale buffer (M * N / 32 bytes). Both fused-quantize GEMMs use
 * MXB200_SCALE_REFERENCE, the only rule the reference's fused kernels have; MXB200_SCALE_OCP_FLOOR exists in the
 * stand-alone quantizer only. */
MXB200_API int mxb200_gemm_relu_square(const void* a, const void* a_scale, const void* b, const void* b_scale, void* h,
                                       void* q, void* q_scale, void* q_t, void* q_t_scale, int64_t M, int64_t N,
                                       int64_t K, void* stream);

/* Replaces nanochat::kernels::cutlass_mx_gemm_relu_square_bwd (mx_gemm_kernel.h:29-32; the MLP backward,
 * fp8.cpp:318-323): ga = bf16(a . b^T) is not written; with h (M, N) bf16 read in the epilogue, the outputs of
 * mxb200_quantize_mx_relu_square_bwd(ga, h), bit for bit: dh (M, N) e4m3 + dh_scale, dh_t (N, M) + dh_t_scale. */
MXB200_API int mxb200_gemm_relu_square_bwd(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                           const void* h, void* dh, void* dh_scale, void* dh_t, void* dh_t_scale,
                                           int64_t M, int64_t N, int64_t K, void* stream);

/* Output kinds of the split-K entry point. */
typedef enum mxb200_out_kind { MXB200_OUT_BF16 = 0, MXB200_OUT_F32 = 1 } mxb200_out_kind;

/* Deterministic split-K for long-K, few-tile shapes (the weight gradients: K = tokens). The K range is cut
 * into `splits` slices run by different CTAs; partial tiles go through `workspace` and are summed in slice
 * order by whichever CTA finishes last, so results do not depend on timing. Counterpart of the reference's
 * split-K choice for these shapes (src/nanochat/model/fp8/mx_gemm.cpp:269-274, 293-314).
 * mxb200_gemm_splits picks a slice count for a shape on the current device (1 = not worth splitting);
 * mxb200_gemm_workspace_bytes gives the bytes `workspace` must hold for that count (0 when splits == 1).
 * The workspace needs no initialisation and may be reused by later calls on the same stream. */
MXB200_API int mxb200_gemm_splits(int64_t M, int64_t N, int64_t K);
MXB200_API size_t mxb200_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int splits);
/* out_kind BF16: d is bf16, resid optional, alpha/accumulate ignored. F32: d is fp32, resid must be null. */
MXB200_API int mxb200_gemm_splitk(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d, int out_kind,
                       const void* resid, int64_t M, int64_t N, int64_t K, const float* alpha, int accumulate,
                       int splits, void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference. mxb200_gemm_splitk for callers that have no device memory to hand over and
 * must not trigger an allocation: a backend wired in at the reference's kernel seam gets plain pointers and a
 * stream but no workspace argument, runs on autograd worker threads in the middle of backward where a
 * cudaMalloc would stall the whole device, and in a trainer whose caching allocator already owns all of HBM a
 * raw allocation simply fails. The partial tiles and tile counters go to an array of
 * MXB200_STATIC_SCRATCH_BYTES that is part of the library's device image (each GPU that loads the library
 * carries it for the life of the process). The call itself allocates nothing, on the device or through any
 * library. Shapes whose mxb200_gemm_workspace_bytes(M, N, K, splits) exceeds that size are refused with
 * MXB200_ERR_WORKSPACE; pick fewer splits or use mxb200_gemm_splitk. The first call on each device looks up
 * the array's device address; make that first call outside any stream capture. All calls on a device share
 * the one array and it keeps whatever the previous call left: the tile counters are cleared on the stream at
 * the start of every call, the partial tiles are fully rewritten before they are read. Two calls whose kernels
 * may overlap on the GPU (different streams, no dependency) would race on it; serialise them. Same arguments
 * and results as mxb200_gemm_splitk, bit for bit. */
#define MXB200_STATIC_SCRATCH_BYTES (32u << 20)
MXB200_API int mxb200_gemm_splitk_static(const void* a, const void* a_scale, const void* b, const void* b_scale, void* d,
                                         int out_kind, const void* resid, int64_t M, int64_t N, int64_t K,
                                         const float* alpha, int accumulate, int splits, void* stream);

/* Static message for a status (the reference's seam returns const char* messages, mx_gemm_kernel.h:12). */
MXB200_API const char* mxb200_strerror(int status);

/* Every device-side wait (GEMM, fused residual step, streaming quantizer) is bounded; a wait that runs out records
 * where in a device word and the kernel returns instead of spinning. This reads that word for the current device
 * (0 = none) and clears it. Synchronises the device. */
MXB200_API int mxb200_device_status(uint32_t* word);

/* Exercises that path without a stuck kernel: launches one warp that waits, with the given limit, on a barrier nothing
 * will ever arrive on, records the give-up as the kernels do (site 0x7f) and returns normally. The next
 * mxb200_device_status then reports MXB200_ERR_WATCHDOG once. limit_ns: 1 to 10 000 000 (10 ms). No reference
 * counterpart: it is how the bounded waits and their reporting are tested. */
MXB200_API int mxb200_selftest_bounded_wait(uint64_t limit_ns, void* stream);

/* Tuning knobs for measurement, process-wide. tile_n: 128 or 256 = the one-CTA kernel with 128 x tile_n tiles;
 * 384 / 512 = the CTA-pair kernel (256 x 192 / 256 x 256 tile over two SMs); 0 = choose per shape. max_ctas: CTAs of the persistent
 * grid (0 = one per SM). Not part of the reference interface. */
MXB200_API int mxb200_set_gemm_config(int tile_n, int max_ctas);

/* How many kernels this library has launched in this process (for benchmark accounting). */
MXB200_API uint64_t mxb200_launch_count(void);

MXB200_API int mxb200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MXB200_H_ */
