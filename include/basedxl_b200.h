/* C ABI of libbasedxl_b200: hand-written sm_100a kernels for the displaced
 * patch-parallel SDXL UNet hot path.
 *
 * The reference project (sekstini/basedxl) is pure Python and has no FFI; each
 * entry point below names the reference code whose device work it replaces
 * (paths are relative to the reference project).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise; tensors are fp16
 *     unless the name says f32; activations are NHWC ("channels last") strips or
 *     [rows, cols] matrices; all strides / leading dimensions are in ELEMENTS
 *   - `stream` is a cudaStream_t passed as void*; calls only enqueue work
 *   - no entry point allocates or frees device memory (bxl_comm_ipc_open / _close map and unmap
 *     a peer process's allocation, at set-up time), none synchronises the host except
 *     bxl_device_status(); workspaces are caller-owned
 *   - return value: 0 = ok, negative = error (see bxl_last_error()); exceptions
 *     never cross this boundary
 *   - one host thread per process drives the library
 */
#ifndef BASEDXL_B200_H
#define BASEDXL_B200_H

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library ------------------------------------------------------------ */

/* Sets up the per-device status word and the TMA descriptor encoder for the
 * current device; fails on anything but compute capability 10.x.
 * Replaces: device selection in BasedXLConfig.__post_init__ (basedxl/utils.py:22-33),
 * without its silent fallback to single-device mode. */
int bxl_init(void);

/* Message of the last failed call on this host thread. */
const char* bxl_last_error(void);

/* Reads (and clears) the device status word that kernels write when a bounded
 * wait gives up.  Blocks the host on a small device->host copy. */
int bxl_device_status(int* code, int* site, int* block);

int bxl_sm_count(void);

/* Launch kernels with programmatic stream serialisation (each kernel's set-up
 * overlaps the tail of the one before it on the stream).  On by default; BXL_PDL=0 in
 * the environment, or this call with 0, turns it off.  No counterpart in the reference. */
int bxl_set_pdl(int enabled);

/* Promise that the B operand of the GEMM entry points and the packed weights of the
 * convolution are never written by the kernel that precedes the launch on its stream (they
 * are model weights).  Their copies then start before the kernel waits for its predecessor,
 * which hides the first fetch from HBM behind the predecessor's tail.  Off by default; the
 * UNet host turns it on.  No counterpart in the reference. */
int bxl_set_static_weights(int enabled);

/* Test hook: force the GEMM / convolution tile width (multiple of 32, <= 256), the K
 * split (1, 2 or 4) and CTA pairing (1 = 256-row tiles on two CTAs, 0 = off); 0 / 0 / -1
 * restore the built-in choice.  No counterpart in the reference. */
int bxl_debug_force_tiles(int bn, int split, int pair);

/* Test hook: force the order in which the convolution's output tiles are handed to the CTAs:
 * 0 = consecutive tiles walk the pixels (they share a weight tile), 1 = they walk the output
 * channels (they share an input tile; chosen by itself when the input exceeds what stays in
 * L2), -1 restores the built-in choice.  No counterpart in the reference. */
int bxl_debug_force_tile_order(int order);

/* Test hook: force the K/V split of the attention kernel (1, 2 or 4 CTAs per query block;
 * 0 restores the built-in choice).  No counterpart in the reference. */
int bxl_debug_force_attn_split(int split);

/* ---- matmul ------------------------------------------------------------- */

/* C[M,N] = A[M,K] * B (+ bias[N]) (+ residual[M,N]); fp16 operands, fp32
 * accumulation in tensor memory, output fp16 (out_f32 = 0) or fp32.
 * b_is_kn = 0: B is [N,K] (an nn.Linear weight as stored).
 * b_is_kn = 1: B is [K,N] row-major (the layout BasedXLLowPLinear keeps).
 * Replaces: cascaded_lowp_matmul / _matmul_kernel
 * (basedxl/triton/cascaded_lowp_matmul.py:54-173), the bias add of
 * BasedXLLowPLinear.forward (basedxl/modules/lowp_linear.py:15-19) and the
 * to_q / to_kv / to_out linears of the attention wrappers
 * (basedxl/modules/attn.py:123,127,159). */
int bxl_gemm_f16(const void* A, long long lda, const void* B, long long ldb, int b_is_kn, const void* bias,
                 const void* residual, long long ldr, void* C, long long ldc, int out_f32, int M, int N, int K,
                 void* stream);

/* One projection, two destinations: [C1 | C2] = A[M,K] * B[N,K]^T + bias[N], the first n1
 * output columns to C1 (row stride ldc1), the remaining N - n1 to C2 (row stride ldc2).
 * n1 must be a multiple of 32.  Used for the fused q | k | v projection of self-attention:
 * q goes to a scratch matrix, k|v straight into this strip's K/V staging slot.
 * Replaces: to_q and to_kv of BasedXLSelfAttentionPP._forward (basedxl/modules/attn.py:123,127)
 * and the staging copy of enqueue (basedxl/utils.py:156). */
int bxl_gemm_dual_f16(const void* A, long long lda, const void* B, long long ldb, const void* bias, void* C1,
                      long long ldc1, int n1, void* C2, long long ldc2, int M, int N, int K, void* stream);

/* Feed-forward input projection with the GEGLU gate fused into the epilogue:
 * h = A[M,K] * B[N,K]^T + bias[N]; out[m, 16c+i] = h[m, 32c+i] * gelu(h[m, 32c+16+i]), i < 16.
 * B and bias are given with their rows INTERLEAVED in groups of 16 value rows followed by
 * the 16 matching gate rows (done once per layer); C is [M, N/2] fp16.  Exact erf GELU.
 * Replaces: the GEGLU projection + chunk + gelu + multiply of the host UNet's feed-forward
 * blocks (the elementwise traffic between the patched operators). */
int bxl_gemm_geglu_f16(const void* A, long long lda, const void* B, long long ldb, const void* bias, void* C,
                       long long ldc, int M, int N, int K, void* stream);

/* General form of the three entry points above (B as [N,K]), with two additions that remove the
 * LayerNorm kernels of the transformer blocks from the step:
 *   - row statistics out: with `row_stats` set, every CTA also writes, per output row, the sum and
 *     the sum of squares of the fp16 values it stored for the column slice it owns:
 *     row_stats[m][part][2] fp32, `*row_stats_parts` partials per row (the count follows from
 *     the tiling chosen for the problem and is at most N/16; row_stats_capacity = floats available);
 *   - LayerNorm folded in: with `ln_partials` set (such partials of the rows of A, `ln_parts` per
 *     row), A is taken as the UN-normalised input of a LayerNorm over K, B as the weight with the
 *     LayerNorm gain multiplied into its columns, `ln_colsum[n]` = sum_k B[n,k] (fp32), and the
 *     bias (`bias_f32`, fp32) as W * beta + b: the epilogue forms
 *     rstd_m * (acc[m,n] - mean_m * ln_colsum[n]) + bias[n], which equals Linear(LayerNorm(A)).
 * Everything else as in bxl_gemm_f16 / bxl_gemm_dual_f16 (C2, ldc2, n_split) / bxl_gemm_geglu_f16
 * (geglu = 1).  Unused pointers are NULL, unused integers 0.
 * Replaces: the LayerNorm -> Linear pairs of the host UNet's transformer blocks (norm1 -> to_q/to_kv,
 * norm2 -> to_q, norm3 -> feed-forward projection) around the attention wrappers
 * (basedxl/modules/attn.py:123,127). */
typedef struct bxl_gemm_fused_args {
  const void* A; long long lda;
  const void* B; long long ldb;
  const void* bias;
  const float* bias_f32;
  const void* residual; long long ldr;
  void* C; long long ldc;
  void* C2; long long ldc2; int n_split;
  int geglu;
  const float* ln_partials; int ln_parts; const float* ln_colsum; float ln_eps;
  float* row_stats; long long row_stats_capacity;
  int M, N, K;
} bxl_gemm_fused_args;
int bxl_gemm_fused_f16(const bxl_gemm_fused_args* args, int* row_stats_parts, void* stream);

/* Split-operand product of fp32 matrices: A[M,K] and B[K,N] (row-major fp32) are
 * each split into fp16 high and low parts and C = Ah*Bh + Ah*Bl + Al*Bh is
 * accumulated in one fp32 tensor-memory accumulator; C is fp32 [M,N].
 * Replaces: the same reference kernel as bxl_gemm_f16, for fp32 operands (the
 * reference's accuracy study, extras/measure_cascaded_lowp_matmul_error.py:12-41). */
long long bxl_gemm_split_workspace_bytes(int M, int N, int K);
int bxl_gemm_split_f32(const float* A, const float* B, float* C, int M, int N, int K, void* workspace,
                       long long workspace_bytes, void* stream);

/* ---- convolution ---------------------------------------------------------- */

/* [C_out][C_in][3][3] -> [C_out][ky][kx][C_in], the weight layout both
 * convolution entry points consume.  Done once per layer at wrap time, like the
 * reference's fused/transposed weight copies (basedxl/modules/lowp_linear.py:12). */
int bxl_conv_weight_pack_f16(const void* w_oihw, void* w_packed, int c_out, int c_in, void* stream);

/* 3x3 convolution, padding 1, stride 1 or 2, of an NHWC H-strip x[B,H_in,W,C_in]
 * whose missing rows above / below come from `top` / `bot` ([B,1,W,C_in], image
 * stride halo_img_stride; NULL = zero row, i.e. the image edge).  Output
 * y[B,H_in/stride,W/stride,C_out] (+ bias[C_out]) (+ bias_rows[B,C_out], rows
 * bias_rows_stride elements apart, 0 = C_out: a slice of a wider matrix that holds the
 * time-embedding projections of several layers) (+ residual, same shape as y).
 * Implicit GEMM on tcgen05; C_in % 64 == 0, C_out % 4 == 0 (the last convolution of the
 * network, 320 -> 4, runs here on a 32-wide tile whose unused weight rows are zero fill).
 * Replaces: BasedConv2dPP.forward's padded-input assembly and F.conv2d
 * (basedxl/modules/conv2d.py:74-104) and naive_forward (:15-18). */
int bxl_conv3x3_halo_f16(const void* x, long long x_img_stride, const void* top, const void* bot,
                         long long halo_img_stride, const void* w_packed, const void* bias, const void* bias_rows,
                         long long bias_rows_stride, const void* residual, void* y, int B, int C_in, int C_out, int H_in,
                         int W, int stride, void* stream);

/* Same contract, stride 1, for the two thin convolutions at the ends of the
 * network (C_in <= 16, or C_out == 4 with C_in % 64 != 0): direct CUDA-core kernels
 * (C_in == 4: four pixels per thread).
 * Replaces: BasedConv2dPP.sliced_forward (basedxl/modules/conv2d.py:20-41) for
 * conv_in, and the forward above for a thin conv_out. */
int bxl_conv3x3_direct_f16(const void* x, long long x_img_stride, const void* top, const void* bot,
                           long long halo_img_stride, const void* w_packed, const void* bias, void* y, int B, int C_in,
                           int C_out, int H, int W, void* stream);

/* First and last `pad` rows of a strip -> out[2][B][pad][W][C].
 * Replaces: the boundary torch.stack (basedxl/modules/conv2d.py:92) and the copy
 * into the staging slot in PatchParallelismCommManager.enqueue (basedxl/utils.py:156). */
int bxl_halo_pack_f16(const void* x, long long img_stride, void* out, int B, int H, int W, int C, int pad, void* stream);

/* ---- GroupNorm -------------------------------------------------------------- */

/* Scratch for bxl_groupnorm_stats_f16.  The first 256 bytes must be zero before
 * the first use and are left zero by every call; calls sharing a scratch buffer
 * must be ordered on one stream. */
long long bxl_groupnorm_scratch_bytes(int B, int G);

/* moments[2][B][G] (fp32): per-group mean and mean of squares of the strip
 * x[B,HW,C].  Replaces: basedxl/modules/groupnorm.py:38-42. */
int bxl_groupnorm_stats_f16(const void* x, long long img_stride, int B, int HW, int C, int G, float* moments,
                            void* scratch, long long scratch_bytes, void* stream);

/* Same result as bxl_groupnorm_stats_f16, for callers that cannot pass scratch
 * memory (hosts that reserved all device memory up front or whose operator
 * callbacks may not call cudaMalloc).  This entry point has no counterpart in the
 * reference.  The scratch is a 262,400-byte array built into the library and
 * resident on every GPU that loads it; it serves B*G <= 256
 * (bxl_groupnorm_stats_noalloc_max_bg()), larger problems are rejected with an
 * error.  Allocates nothing.  The first call on each device looks up the array's
 * device address and should therefore be made before any stream capture begins.
 * All calls share the one array: two calls whose kernels may overlap on the GPU
 * (different streams without ordering) race. */
long long bxl_groupnorm_stats_noalloc_max_bg(void);
int bxl_groupnorm_stats_noalloc_f16(const void* x, long long img_stride, int B, int HW, int C, int G, float* moments,
                                    void* stream);

/* y = GroupNorm(x) (* sigmoid, if silu) using
 *   mode 0: the strip's own moments                         (groupnorm.py:44-45)
 *   mode 1: the average of all peers' fresh moments         (groupnorm.py:46-48)
 *   mode 2: average of stale peer moments + fresh - stale own (groupnorm.py:49-52)
 * followed by the reference's negative-variance fallback and local-count Bessel
 * factor (groupnorm.py:56-63) and the affine map (:64-69).
 * peer_moments: HOST array of n_peers device pointers, each [2][B][G] fp32; in
 * mode 1 entry `own` is ignored (the fresh moments are used). */
int bxl_groupnorm_apply_f16(const void* x, void* y, long long img_stride, int B, int HW, int C, int G,
                            const float* fresh_moments, const float* const* peer_moments, int n_peers, int own, int mode,
                            float eps, const void* gamma, const void* beta, int silu, void* stream);

/* GroupNorm (+ SiLU) in ONE launch for the local (mode 0) and stale (mode 2) cases: a cluster of
 * thread blocks per (image, run of whole groups) reads the strip x[B,H,W,C] once, keeps it in
 * shared memory while the group sums are exchanged inside the cluster, and normalises it from
 * there.  Same arithmetic as bxl_groupnorm_stats_f16 followed by bxl_groupnorm_apply_f16.
 * fresh_out (or NULL): [2][B][G] fp32 moments of this strip; it may be the strip's own entry of
 * peer_moments (its staging range): the stale values are read before the fresh ones are stored.
 * halo_out (or NULL): [2][B][W][C] fp16, the first and the last pixel row of y - the rows the
 * 3x3 convolution that consumes y publishes to the neighbouring strips (conv2d.py:92).
 * The synchronous mode (fresh moments of all strips) needs a collective between the two passes
 * and stays on the two-launch form.
 * Replaces: BasedXLGroupNorm.forward (basedxl/modules/groupnorm.py:38-69) without a collective,
 * the staging copy of its moments and of the following convolution's boundary rows
 * (basedxl/utils.py:156). */
int bxl_groupnorm_fused_f16(const void* x, void* y, long long img_stride, int B, int H, int W, int C, int G,
                            float* fresh_out, const float* const* peer_moments, int n_peers, int own, int mode, float eps,
                            const void* gamma, const void* beta, int silu, void* halo_out, void* stream);

/* ---- attention ---------------------------------------------------------------- */

/* out[b, l, h*64 + d] = softmax_l'(q . k * scale) v over the concatenation of
 * n_slots key/value slots, each [B, L_slot, ld_kv] with K of head h at columns
 * h*64 and V at v_col0 + h*64.  kv_slots: HOST array of n_slots device pointers
 * (slot order = token order).  Head dimension 64.
 * Replaces: the KV concatenation, split, head reshapes and
 * F.scaled_dot_product_attention of BasedXLSelfAttentionPP._forward
 * (basedxl/modules/attn.py:129-156) and of BasedXLCrossAttentionPP.forward
 * (basedxl/modules/attn.py:79-91). */
int bxl_attn_fwd_f16(const void* q, long long q_img_stride, long long ld_q, const void* const* kv_slots, int n_slots,
                     long long kv_img_stride, long long ld_kv, int v_col0, void* out, long long out_img_stride,
                     long long ld_out, int B, int heads, int L_q, int L_slot, float scale, void* stream);

/* ---- exchange between strips over peer memory ----------------------------------- */

/* Size of a group's control words (sequence-number flags; see bxl_comm_exchange).  The caller
 * allocates them ZEROED in memory that every peer of the group can write, one block per rank. */
long long bxl_comm_ctl_bytes(void);

/* Mapping a buffer of a peer process (same node) into this one, for bxl_comm_exchange.
 * bxl_comm_ipc_export: the 64-byte CUDA IPC handle of the allocation that contains `ptr` (any
 *   cudaMalloc-backed device memory of this process, e.g. a framework tensor) and ptr's offset in it;
 *   the owner keeps the memory allocated while peers have it open.
 * bxl_comm_ipc_open: maps that allocation for kernels of the CURRENT device (which also switches on
 *   peer access between the two devices) and returns its base address in this process; the peer's
 *   buffer is at base + offset.  An allocation can be opened once per process.
 * bxl_comm_ipc_close: unmaps it.
 * The three calls are set-up time; they are the only entry points that touch the address space.
 * No counterpart in the reference (its collectives leave transport set-up to NCCL). */
int bxl_comm_ipc_export(const void* ptr, unsigned char* handle64, long long* offset_bytes);
int bxl_comm_ipc_open(const unsigned char* handle64, void** base_out);
int bxl_comm_ipc_close(void* base);

/* What a blocking all-gather of one contribution per rank does, as ONE kernel over peer memory
 * (NVLink): copies `nbytes` from `src` (this rank's memory) to peer_dst[p] for every p with a
 * non-NULL entry (the place of this rank's contribution in peer p's memory, mapped into this
 * process; entry `own` may be NULL when src already is that place), then meets the peers at a
 * flag barrier, so that when the kernel ends every peer's contribution has arrived in THIS
 * rank's memory.  ctl = this rank's control words, peer_ctl[p] = peer p's (mapped); peer_dst and
 * peer_ctl are HOST arrays of n_peers device pointers.  All ranks of a group launch the same
 * sequence of exchanges, each rank on one stream.  handshake != 0: first wait until every peer has
 * reached this exchange, for a destination that the previous exchange of the group also wrote
 * (the per-step output).  Waits give up after wait_seconds and report through
 * bxl_device_status() (site 800 + peer: handshake, 900 + peer: arrival).
 * Replaces: the blocking per-layer dist.all_gather of the synchronous steps
 * (basedxl/modules/conv2d.py:95, groupnorm.py:47, attn.py:135) and the output gather
 * (basedxl/unet.py:172,193). */
int bxl_comm_exchange(const void* src, void* const* peer_dst, long long nbytes, void* ctl, void* const* peer_ctl,
                      int n_peers, int own, int handshake, double wait_seconds, void* stream);

/* ---- host-graph helpers (the elementwise work between the patched operators) -- */

/* y[B,2H,2W,C] = nearest-neighbour up-sampling of x[B,H,W,C]. */
int bxl_upsample2x_f16(const void* x, void* y, int B, int H, int W, int C, void* stream);
/* LayerNorm over the last axis of x[rows,C]. */
int bxl_layernorm_f16(const void* x, void* y, const void* gamma, const void* beta, long long rows, int C, float eps,
                      void* stream);
/* out[rows,F] = h[:, :F] * gelu(h[:, F:]) for h[rows,2F] (exact erf GELU). */
int bxl_geglu_f16(const void* h, void* out, long long rows, int F, void* stream);

/* One kernel for what follows the UNet in every denoising step: classifier-free guidance
 * eps = eps_u + g (eps_c - eps_u) on eps[2][n] (fp16), the Euler update
 * latents += eps * (sigma_next - sigma) in fp32 (in place), and the next model input
 * next_input[2][n] = latents / sqrt(sigma_next^2 + 1) (fp16, both CFG rows).
 * Replaces: the guidance combine and scheduler step the denoising loop runs around
 * BasedXLUnet.forward (the loop of basedxl/model.py:39-45 / sample.py:68-75). */
int bxl_cfg_euler_step(const void* eps, float* latents, void* next_input, long long n, float guidance, float sigma,
                       float sigma_next, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BASEDXL_B200_H */
