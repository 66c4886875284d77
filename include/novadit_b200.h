/*
 * novadit_b200 — C ABI of the B200 (sm_100a) DiT operator kernels.
 *
 * Plain pointers and sizes only: no torch types, no exceptions, no allocation,
 * no synchronisation. Every entry point validates its arguments, enqueues its
 * kernels on `stream` (a cudaStream_t passed as void*; NULL = the legacy
 * default stream) of the CURRENT device and returns ND_OK or a negative
 * nd_status. All pointers are device pointers on that device unless stated.
 *
 * Row sharding: the row operators see `rows` consecutive rows of the
 * flattened [B*S, H] activation starting at global row `row_start`; sample
 * index b = (row_start + r) / seq_len selects the modulation vector, so
 * `scale` / `shift` / `dscale` / `dshift` always point at the FULL [B, H]
 * arrays while x / y / dy / dx / statistics point at the local shard.
 *
 * Each declaration cites the interface of the NovaDiT reference it replaces
 * (path inside that project : line).
 */
#ifndef NOVADIT_B200_H_
#define NOVADIT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
enum {
  ND_OK = 0,
  ND_ERR_BAD_ARG = -1,     /* null pointer, negative size, inconsistent shape */
  ND_ERR_UNSUPPORTED = -2, /* dtype / size outside what the kernels cover */
  ND_ERR_LAUNCH = -3,      /* CUDA reported an error at launch; see nd_last_cuda_error() */
  ND_ERR_WORKSPACE = -4,   /* workspace missing, too small or misaligned */
  ND_ERR_DEVICE = -5,      /* a bounded device-side wait expired (see the status argument of nd_fc1_fwd) */
  ND_ERR_TOO_LARGE = -6    /* the problem needs more scratch than the no-allocation entry point carries */
};

/* element types. csrc/common/type_dispatch.h:5-6 dispatches on the same set */
enum { ND_F16 = 0, ND_BF16 = 1, ND_F32 = 2, ND_E4M3 = 3 };

/* activation ids: csrc/common/dispatch.h:7-10 (kSilu = 0, kGelu = 1; GELU is the tanh form) */
enum { ND_ACT_SILU = 0, ND_ACT_GELU = 1, ND_ACT_NONE = 2 /* identity: nd_fc1_fwd with gated == 0 only */ };

const char* nd_status_string(int status);
/* cudaError_t of the last failed launch on the calling thread (0 if none) */
int nd_last_cuda_error(void);
int nd_version(void);
/* Error word of the current device: 0, or the code a kernel left when one of its bounded waits
 * expired (1..3: a norm kernel waiting for a bulk copy into shared memory; 101..114: an FC1 kernel
 * waiting for an operand stage, an accumulator or a dy block - its output is then incomplete).
 * Covers every kernel of the library, including launches made through the torch extension, which
 * passes no status word of its own. Synchronises with the device (a blocking copy).
 * reset != 0 clears it. Negative = nd_status of a failed query. */
int nd_device_error(int reset);

/* ------------------------------------------------------------------ AdaLN */

/* y = LN(x) * (1 + scale[b]) + shift[b]; writes fp32 mean / invstd per row when
 * both pointers are non-null (training) and skips them when both are null
 * (inference). dtype: ND_F16, ND_BF16 or ND_F32 (x, scale, shift, y share it).
 * Replaces fused_adaln_{fp16,bf16}_ungated_forward and the inference variants,
 * csrc/ops/adaln_kernel.cu:960-1020, called from fused_adaln_forward :1022-1073
 * and fused_adaln_forward_inference :1075-1145. */
int nd_adaln_fwd(int dtype, const void* x, const void* scale, const void* shift, void* y,
                 float* mean, float* invstd, int64_t rows, int64_t row_start, int64_t seq_len,
                 int64_t hidden, float eps, void* stream);

/* AdaLN / AdaRMSNorm forward with FP8 e4m3 OUTPUT for an FP8 consumer (nd_fc1_fwd with ND_E4M3 operands):
 * q [rows, hidden] bytes = saturate_e4m3(y / *q_scale), statistics as in the 16-bit forward, and, when `amax` is
 * not NULL, *amax = max(*amax, max |y|) over the launch (exact, order-independent). Delayed scaling: the caller
 * passes the scale derived from an earlier step's maximum (amax / 448) and reads this step's maximum for the
 * next one, so the activation never exists in 16 bits and no separate amax / quantise pass runs. q_scale and amax
 * are device floats. Rows up to 192 16-byte vectors wide (hidden <= 1536 for 16-bit inputs), 16-byte aligned;
 * anything else returns ND_ERR_UNSUPPORTED. No counterpart in the reference (it has no FP8 path). */
int nd_adaln_fwd_e4m3(int dtype, const void* x, const void* scale, const void* shift, void* q, float* mean,
                      float* invstd, const float* q_scale, float* amax, int64_t rows, int64_t row_start,
                      int64_t seq_len, int64_t hidden, float eps, void* stream);
int nd_adarms_fwd_e4m3(int dtype, const void* x, const void* scale, const void* shift, void* q,
                       float* inv_rms, const float* q_scale, float* amax, int64_t rows, int64_t row_start,
                       int64_t seq_len, int64_t hidden, float eps, void* stream);

/* AdaLN / AdaRMSNorm forward with the gated residual of the block in front, in ONE pass:
 *   x_new = x + gate[b] * branch   (gate NULL: x + branch), rounded once to the element type and written out,
 *   y     = norm(x_new) * (1 + scale[b]) + shift[b], statistics of x_new as in nd_adaln_fwd.
 * Bytes moved: 4 tensors of [rows, hidden] (x, branch in; x_new, y out) instead of the 5 of a residual kernel
 * followed by a norm kernel; results are bit-identical to that composition (nd_gated_residual_fwd or
 * nd_out_residual_fwd, then nd_adaln_fwd), which is also what runs for rows the one-pass kernel does not take
 * (not 16-byte vectorisable, or wider than 512 vectors). The operators are specified in the reference
 * (SPEC.md:293-376, novadit/ops/residual.py:8-25) but it has no fused kernel: no counterpart there. Backward:
 * nd_adaln_bwd on x_new, then nd_gated_residual_bwd_add, which adds the residual stream's own gradient. */
int nd_adaln_fwd_residual(int dtype, const void* x, const void* branch, const void* gate, const void* scale,
                          const void* shift, void* x_new, void* y, float* mean, float* invstd, int64_t rows,
                          int64_t row_start, int64_t seq_len, int64_t hidden, float eps, void* stream);
int nd_adarms_fwd_residual(int dtype, const void* x, const void* branch, const void* gate, const void* scale,
                           const void* shift, void* x_new, void* y, float* inv_rms, int64_t rows, int64_t row_start,
                           int64_t seq_len, int64_t hidden, float eps, void* stream);

/* dx = invstd * (dxhat - mean_h(dxhat) - xhat * mean_h(dxhat * xhat)), dxhat = dy * (1 + scale[b]).
 * Replaces the launcher behind fused_adaln_backward_dx, csrc/ops/adaln_kernel.cu:1147-1193
 * (kernel :473-582). */
int nd_adaln_bwd_dx(int dtype, const void* dy, const void* x, const void* scale,
                    const float* mean, const float* invstd, void* dx, int64_t rows,
                    int64_t row_start, int64_t seq_len, int64_t hidden, void* stream);

/* Bytes of scratch the dparam / fused backward entry points need for this shard: fp32 partial
 * column sums, no counters, nothing to initialise. The base must be 256-byte aligned. One
 * workspace serves one launch at a time (launches on one stream may share it). */
size_t nd_norm_dparam_ws_bytes(int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden);

/* dscale[b,h] = sum_s dy * xhat, dshift[b,h] = sum_s dy over the shard's rows of
 * sample b, fp32, for every sample the shard touches (other rows of dscale /
 * dshift are left untouched). Two-stage and deterministic: fp32 partials per
 * row segment in `ws`, then a second kernel sums them in index order (no atomics).
 * Replaces the launcher behind fused_adaln_backward_dparam,
 * csrc/ops/adaln_kernel.cu:1195-1245 (kernel :584-615). */
int nd_adaln_bwd_dparam(int dtype, const void* dy, const void* x, const float* mean,
                        const float* invstd, float* dscale, float* dshift, int64_t rows,
                        int64_t row_start, int64_t seq_len, int64_t hidden, void* ws,
                        size_t ws_bytes, void* stream);

/* dx and dscale/dshift in ONE pass over dy and x (what the autograd backward of
 * novadit/ops/adaln.py:25-47 needs when every input wants a gradient; the
 * reference launches the two kernels above one after the other). */
int nd_adaln_bwd(int dtype, const void* dy, const void* x, const void* scale, const float* mean,
                 const float* invstd, void* dx, float* dscale, float* dshift, int64_t rows,
                 int64_t row_start, int64_t seq_len, int64_t hidden, void* ws, size_t ws_bytes,
                 void* stream);

/* nd_adaln_bwd for callers that cannot provide scratch memory (no counterpart in the reference).
 * Who needs it: a process that handed all device memory to its own pool at start-up, a plugin whose
 * host forbids allocations, code inside a stream capture or a latency-critical loop where cudaMalloc
 * is illegal or stalls the device. The fp32 partial sums of the dparam reduction go through a fixed
 * array of nd_noalloc_scratch_bytes() (16 MiB) in the library's own device image, which every GPU
 * that loads the library holds until the process exits; inputs and outputs are still the caller's.
 * The call allocates nothing and calls no allocating routine. Problems whose
 * nd_norm_dparam_ws_bytes(...) exceeds the array are refused with ND_ERR_TOO_LARGE (use nd_adaln_bwd
 * with your own workspace). The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and should come before any stream capture. It is
 * also the call that makes the CUDA runtime load the array and the kernels onto that device (modules load
 * lazily): a process that later hands all free device memory to its own pool should make one small
 * warm-up call per device at start-up, before it does so, or that first call fails with ND_ERR_LAUNCH. All
 * calls on a device share the one array: calls whose kernels may overlap on the GPU (different
 * streams) race on it and must be serialised by the caller. The array keeps the previous call's
 * contents; nothing in it needs clearing. Same arguments and results as nd_adaln_bwd. */
size_t nd_noalloc_scratch_bytes(void);
int nd_adaln_bwd_noalloc(int dtype, const void* dy, const void* x, const void* scale, const float* mean,
                         const float* invstd, void* dx, float* dscale, float* dshift, int64_t rows,
                         int64_t row_start, int64_t seq_len, int64_t hidden, void* stream);

/* ------------------------------------------------------------- AdaRMSNorm */

/* y = x * inv_rms * (1 + scale[b]) + shift[b], inv_rms = 1/sqrt(mean(x^2) + eps);
 * inv_rms nullable (inference). Replaces fused_adarmsnorm_{fp16,bf16}_forward,
 * csrc/ops/adarmsnorm_kernel.cu:928-961 (entry points :965-1060). */
int nd_adarms_fwd(int dtype, const void* x, const void* scale, const void* shift, void* y,
                  float* inv_rms, int64_t rows, int64_t row_start, int64_t seq_len,
                  int64_t hidden, float eps, void* stream);

/* dx = inv_rms * (dxhat - xhat * mean_h(dxhat * xhat)). Replaces
 * fused_adarmsnorm_backward_dx, csrc/ops/adarmsnorm_kernel.cu:457-565. */
int nd_adarms_bwd_dx(int dtype, const void* dy, const void* x, const void* scale,
                     const float* inv_rms, void* dx, int64_t rows, int64_t row_start,
                     int64_t seq_len, int64_t hidden, void* stream);

/* Replaces fused_adarmsnorm_backward_dparam, csrc/ops/adarmsnorm_kernel.cu:571-600. */
int nd_adarms_bwd_dparam(int dtype, const void* dy, const void* x, const float* inv_rms,
                         float* dscale, float* dshift, int64_t rows, int64_t row_start,
                         int64_t seq_len, int64_t hidden, void* ws, size_t ws_bytes,
                         void* stream);

/* One-pass dx + dscale/dshift (autograd backward of novadit/ops/adarmsnorm.py:25-47). */
int nd_adarms_bwd(int dtype, const void* dy, const void* x, const void* scale,
                  const float* inv_rms, void* dx, float* dscale, float* dshift, int64_t rows,
                  int64_t row_start, int64_t seq_len, int64_t hidden, void* ws, size_t ws_bytes,
                  void* stream);

/* --------------------------------------------------------------- gate-act */

/* x rows are [up(I) | gate(I)]; y = up * act(gate). dtype ND_F16 / ND_BF16 / ND_F32.
 * Replaces fused_gate_act_{fp32,fp16,bf16}_forward, csrc/ops/gate_act_kernel.cu:536-600
 * (entry points fused_gate_act_forward / fused_geglu_forward :604-721). */
int nd_gate_act_fwd(int dtype, int act, const void* x, void* y, int64_t rows, int64_t inter,
                    void* stream);

/* dz = [dy * act(gate) | dy * up * act'(gate)], rows of 2I. Replaces the launchers behind
 * fused_gate_act_backward / fused_geglu_backward, csrc/ops/gate_act_kernel.cu:723-857. */
int nd_gate_act_bwd(int dtype, int act, const void* dy, const void* x, void* dz, int64_t rows,
                    int64_t inter, void* stream);

/* The same backward for rows laid out [gate(I) | up(I)]: FC1's pre-activation z = x W^T + b with the
 * nn.Linear weight as stored (gate block first), dz = [dy * up * act'(gate) | dy * act(gate)]. Replaces
 * the eager PyTorch activation backward of the reference's FC1 autograd Function,
 * novadit/ops/fc1_bias_act.py:255-270. */
int nd_gate_act_bwd_gate_first(int dtype, int act, const void* dy, const void* z, void* dz,
                               int64_t rows, int64_t inter, void* stream);

/* --------------------------------------------------------------- row operators next to the path */

/* y = x + residual (+ bias[h]) over [rows, hidden]; fp32 sum, one rounding. dtype ND_F16 / ND_BF16 /
 * ND_F32; bias may be NULL. The reference specifies this operator (novadit/ops/residual.py:8-25,
 * binding fused_out_residual_forward csrc/bindings.cpp:93) but its kernel is a stub that raises
 * (csrc/ops/residual_kernel.cu:3-8). */
int nd_out_residual_fwd(int dtype, const void* x, const void* residual, const void* bias, void* y,
                        int64_t rows, int64_t hidden, void* stream);

/* Rows of qkv [rows, 3*hidden] split into q, k, v [rows, hidden] (hidden = heads * head_dim, so the
 * outputs are the contiguous [B, S, heads, head_dim] tensors of novadit/ops/qkv_pack.py:9-23), and the
 * inverse for the backward pass. Binding fused_qkv_pack_forward csrc/bindings.cpp:91; the reference's
 * kernel is a stub that raises (csrc/ops/qkv_pack_kernel.cu:5-10). */
int nd_qkv_pack_fwd(int dtype, const void* qkv, void* q, void* k, void* v, int64_t rows,
                    int64_t hidden, void* stream);
int nd_qkv_pack_bwd(int dtype, const void* dq, const void* dk, const void* dv, void* dqkv,
                    int64_t rows, int64_t hidden, void* stream);

/* Gated residual of adaLN-Zero DiT blocks (the harness of workload config 5; no counterpart in the reference,
 * whose block has no gate): y = x + gate[b, :] * branch for rows of sample b = (row_start + r) / seq_len, gate
 * [batch, hidden]. Backward: dbranch = gate * dy, and dgate_partials [samples_in_shard * tiles, hidden] fp32 =
 * column sums of dy * branch per tile of `tile_rows` rows of a sample (tiles = ceil(seq_len / tile_rows)); the
 * caller sums the tiles of a sample in order. dx of the residual is dy itself. nd_gated_residual_ws_bytes gives
 * the size of the partials. */
int nd_gated_residual_fwd(int dtype, const void* x, const void* branch, const void* gate, void* y, int64_t rows,
                          int64_t row_start, int64_t seq_len, int64_t hidden, void* stream);
size_t nd_gated_residual_ws_bytes(int64_t rows, int64_t row_start, int64_t seq_len, int64_t hidden,
                                  int64_t tile_rows);
int nd_gated_residual_bwd(int dtype, const void* dy, const void* branch, const void* gate, void* dbranch,
                          float* dgate_partials, int64_t rows, int64_t row_start, int64_t seq_len,
                          int64_t hidden, int64_t tile_rows, void* stream);
/* The same with a second gradient of the residual sum added first: dsum = dy + dres (rounded once, written out:
 * the gradient that flows on along the residual stream), dbranch = gate * dsum, partials of dsum * branch. It
 * replaces the separate addition of the two gradients that reach x_new of nd_adaln_fwd_residual (from the norm
 * and from the stream). No counterpart in the reference. */
int nd_gated_residual_bwd_add(int dtype, const void* dy, const void* dres, const void* branch, const void* gate,
                              void* dsum, void* dbranch, float* dgate_partials, int64_t rows, int64_t row_start,
                              int64_t seq_len, int64_t hidden, int64_t tile_rows, void* stream);

/* -------------------------------------------------------------------- FC1 */

/* z = (x @ w^T) * alpha + bias, x [m,k] and w [n,k] both K-contiguous (nn.Linear layout).
 *   gated == 1: rows [0, n/2) of w (and bias) are the gate, [n/2, n) the value;
 *               y [m, n/2] = value * act(gate)  (layout of novadit/ops/fc1_bias_act.py:55-68).
 *   gated == 2: same function, rows interleaved (gate0, value0, gate1, ...): the layout
 *               fused_fc1_bias_act_forward receives from novadit/ops/fc1_bias_act.py:237-239.
 *   gated == 0: y [m, n] = act(z); with act == ND_ACT_NONE a plain GEMM + bias, which is how the
 *               backward dx = dz @ W of the reference's FC1GatedActSM120BF16BackwardDxKernel
 *               (csrc/cute_dsl/fc1_bias_act/fc1_bias_act.py:996-1913, called from
 *               novadit/ops/fc1_bias_act.py:288-326) runs here: x := dz, w := W^T.
 * ab_dtype: ND_BF16, ND_F16 or ND_E4M3 (both operands); out_dtype: ND_BF16 or ND_F16, also the
 * dtype of `bias` (nullable, length n). alpha = alpha_host * (alpha_dev ? alpha_dev[0] *
 * alpha_dev[1] : 1): pass the two per-tensor de-quantisation scales of an FP8 call as a
 * 2-float device array so no host round trip is needed. fp32 accumulation in tensor memory.
 * Needs k % 16 == 0 bytes-aligned rows (k*sizeof(ab) % 16 == 0) and 16-byte aligned bases.
 * `status` is a device int the kernel sets non-zero if a bounded wait expires (nullable).
 * Replaces fused_fc1_bias_act_forward, csrc/ops/fc1_bias_act_kernel.cu:54-72 (a stub that
 * raises), and the launch of the CuTe-DSL kernel, novadit/ops/fc1_bias_act.py:227-235 with
 * csrc/cute_dsl/fc1_bias_act/aot_bridge.h:17-37 as the intended C signature. */
int nd_fc1_fwd(int ab_dtype, int out_dtype, int act, int gated, const void* x, const void* w,
               const void* bias, float alpha_host, const float* alpha_dev, void* y, int64_t m,
               int64_t k, int64_t n, int* status, void* stream);

/* Backward of the fused FC1 with respect to its pre-activation, recomputation included:
 * dz [m, n] = [dy * value * act'(gate) | dy * act(gate)] with [gate | value] = x @ w^T + bias for w rows
 * [gate block | value block] (gated == 1 of nd_fc1_fwd), dy [m, n/2]. One launch of the forward
 * kernel's main loop with the activation backward as epilogue; z is never written. dtype ND_BF16 or
 * ND_F16 for x, w, bias, dy and dz. Replaces F.linear + the eager activation backward of
 * novadit/ops/fc1_bias_act.py:255-270. `status` as in nd_fc1_fwd. */
int nd_fc1_bwd_dz(int dtype, int act, const void* x, const void* w, const void* bias, const void* dy,
                  void* dz, int64_t m, int64_t k, int64_t n, int* status, void* stream);

/* nd_fc1_bwd_dz that also returns dbias [n] = the sum of dz over the m tokens (of the values as stored, i.e. rounded
 * to the element type, accumulated in fp32 in a fixed order: the `dz_flat.sum(dim=0)` of
 * novadit/ops/fc1_bias_act.py:279) without reading dz again: each epilogue warp leaves the column sums of its 32
 * rows in `ws` (nd_fc1_bwd_dbias_ws_bytes(m, n) bytes, 16-byte aligned, no initialisation needed), a second small
 * launch adds them in row order. dbias has the element type of dz. */
size_t nd_fc1_bwd_dbias_ws_bytes(int64_t m, int64_t n);
int nd_fc1_bwd_dz_dbias(int dtype, int act, const void* x, const void* w, const void* bias, const void* dy,
                        void* dz, void* dbias, void* ws, size_t ws_bytes, int64_t m, int64_t k, int64_t n,
                        int* status, void* stream);

/* The two GEMMs of the FC1 backward on the tcgen05 path, fp32 accumulation, operands read where they lie (UMMA
 * takes W and, for dW, dz as MN-major operands: no transpose copy per call, unlike the reference's
 * _backward_dx_cute, novadit/ops/fc1_bias_act.py:309-315, which copies and transposes both weight halves):
 *   op 0: c [m, n] = a [m, k] @ b [k, n]       dx = dz @ W    (m tokens, k = 2I, n = H): the job of
 *         FC1GatedActSM120BF16BackwardDxKernel, csrc/cute_dsl/fc1_bias_act/fc1_bias_act.py:996-1913
 *   op 1: c [m, n] = a [k, m]^T @ b [k, n]     dW = dz^T @ x  (m = 2I, k tokens, n = H): replaces the
 *         `dz_flat.T @ x_flat` of novadit/ops/fc1_bias_act.py:276
 * fp16 / bf16, all three matrices row-major and dense; n (and k for op 0, m for op 1) a multiple of 8, bases
 * 16-byte aligned, else ND_ERR_UNSUPPORTED. `status` as in nd_fc1_fwd.
 * `ws` (nd_fc1_bwd_gemm_ws_bytes() bytes, 256-byte aligned, no initialisation needed, may be shared by launches
 * on one stream) lets the launch cut the reduction dimension evenly over the GPU: 256 x 256 tiles on CTA pairs
 * (tcgen05 cta_group::2), the k-blocks of all tiles laid end to end and shared out in equal ranges, a tile cut
 * between two pairs finished by whichever of the two comes second from fp32 partials in `ws`; the result does not
 * depend on which. With ws == NULL (or too small) the launch falls back to whole 128 x 192 tiles per CTA, which
 * leaves the last round of tiles partly empty at DiT shapes. */
size_t nd_fc1_bwd_gemm_ws_bytes(void);
int nd_fc1_bwd_gemm(int dtype, int op, const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                    void* ws, size_t ws_bytes, int* status, void* stream);

/* out [cols] = column sums of x [rows, cols] (fp16 / bf16, cols a multiple of 8) with fp32 accumulation in a fixed
 * order (two stages through `ws`, nd_colsum_ws_bytes(cols) bytes, 16-byte aligned): dbias = sum of dz over the
 * tokens, the `dz_flat.sum(dim=0)` of novadit/ops/fc1_bias_act.py:279. */
size_t nd_colsum_ws_bytes(int64_t cols);
int nd_colsum(int dtype, const void* x, int64_t rows, int64_t cols, void* out, void* ws, size_t ws_bytes,
              void* stream);

/* amax = max |x| over n elements (fp32 result, device). Two-stage and deterministic:
 * `ws` holds per-CTA maxima; nd_amax_ws_bytes() bytes, 256-byte aligned. No counterpart in
 * the reference (it has no FP8 path). */
size_t nd_amax_ws_bytes(void);
int nd_amax(int dtype, const void* x, int64_t n, float* amax, void* ws, size_t ws_bytes,
            void* stream);

/* q = saturate_e4m3(x * 448 / amax), scale_out[0] = amax / 448 (1 if amax == 0); amax and
 * scale_out are device floats. No counterpart in the reference. */
int nd_quant_e4m3(int dtype, const void* x, int64_t n, const float* amax, void* q,
                  float* scale_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NOVADIT_B200_H_ */
