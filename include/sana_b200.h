/* C ABI of libsana_b200: the B200 (sm_100a) kernels behind the Sana Linear-DiT block.
 *
 * Upstream (NVlabs/Sana) has no C/FFI plugin interface for this path; its seams are the
 * Python modules LiteLA / GLUMBConv / SanaMSBlock.  Each entry point below names the
 * upstream Python statement(s) it replaces.  The torch-side glue (sana_b200/ops.py) is the
 * only caller: it passes raw device pointers, sizes in elements, and the current CUDA
 * stream.
 *
 * Conventions
 *  - every pointer is a device pointer unless stated otherwise; the caller owns all memory
 *    (inputs, outputs, workspaces); unless an entry point says otherwise the library
 *    allocates nothing on the device and keeps no device state;
 *  - all tensors are token-major ("channels last"): a [T, C] activation is T rows of C
 *    contiguous elements with a row stride given in ELEMENTS (ld*);
 *  - `stream` is a cudaStream_t passed as void*; every call is asynchronous on it;
 *  - return value: 0 = ok; <0 = invalid argument detected on the host before any launch;
 *    >0 = a CUDA runtime error code.  sana_last_error() returns a message for the last
 *    non-zero status on the calling thread.  Nothing throws or exits across this boundary.
 */
#ifndef SANA_B200_H_
#define SANA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SANA_OK 0
#define SANA_ERR_INVALID (-1)
#define SANA_ERR_UNSUPPORTED (-2)
#define SANA_ERR_DRIVER (-3)

/* element types of activations / weights */
#define SANA_F32 0
#define SANA_BF16 1

/* library ABI version (bumped when a signature changes) */
int sana_abi_version(void);
/* message for the last failing call on this thread ("" if none) */
const char* sana_last_error(void);

/* ---------------------------------------------------------------------------------------
 * adaLN-single LayerNorm + modulate:  z = LN(x) * (1 + scale_b) + shift_b
 *   scale_b[c] = table[scale_row, c] + t[b, scale_row*C + c]   (same for shift_row)
 * Replaces `t2i_modulate(self.norm1(x), shift_msa, scale_msa)` and the norm2 twin,
 * diffusion/model/nets/sana_multi_scale.py:148-155 with sana_blocks.py:44-45; LayerNorm is
 * affine-free with biased variance and eps (1e-6 in the block).
 *   x, z  [B*N, C] (row stride C);  table [6, C];  t [B, 6*C];  all of `dtype`.
 * Statistics and the modulation are computed in fp32, one rounding on store.
 * C must be a multiple of 8 and one row at most 16 KiB (8192 bf16 / 4096 fp32 channels).
 */
int sana_ln_modulate(const void* x, const void* table, const void* t, void* z, int64_t B, int64_t N,
                     int64_t C, int shift_row, int scale_row, float eps, int dtype, void* stream);

/* Same kernel with the rows of `table` and of `t` named separately, for modulation layouts
 * other than the block's [6, C] / [B, 6*C]:  scale_b = table[table_scale_row] +
 * t[b, t_scale_row] with table [table_rows, C] and t [B, t_rows, C] (same for shift).
 * Replaces `T2IFinalLayer.forward` up to its linear (sana_blocks.py:919-925):
 * `t2i_modulate(norm_final(x), shift, scale)` with (shift, scale) =
 * (scale_shift_table[None] + t[:, None]).chunk(2, dim=1), i.e. table_rows = 2, t_rows = 1. */
int sana_ln_modulate_rows(const void* x, const void* table, const void* t, void* z, int64_t B, int64_t N,
                          int64_t C, int table_rows, int table_shift_row, int table_scale_row, int t_rows,
                          int t_shift_row, int t_scale_row, float eps, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * RMSNorm with weight over the channel dimension:  y = weight * x * rsqrt(mean_c(x^2) + eps)
 * Replaces `self.q_norm(q)` / `self.k_norm(k)` of LiteLA (qk_norm=True; RMSNorm over the full
 * C, diffusion/model/nets/sana_blocks.py:238-243,274-275 with norms.py:216-231) and of the
 * cross-attention (cross_norm=True, sana_blocks.py:62-64,77-78).
 *   x, y [rows, C] with row strides ldx / ldy in elements (column slices of the qkv / kv
 *   projections are fine; y may alias x); weight [C].  fp32 statistics, one rounding on store.
 */
int sana_rmsnorm(const void* x, int64_t ldx, const void* weight, void* y, int64_t ldy, int64_t rows,
                 int64_t C, float eps, int dtype, void* stream);

/* Rotary embedding of q or k, in place, before the ReLU feature map: replaces
 * `apply_rotary_emb(q, rotary_emb, use_real_unbind_dim=-2)` in `LiteLA.forward`
 * (sana_blocks.py:282-284 with :1549-1586): channel pairs (2i, 2i+1) of every head,
 * y = x * cos + rot(x) * sin in fp32, rounded once to `dtype`.
 *   x [B*N, C] view (row stride ld), e.g. the q or k column block of the qkv projection;
 *   cos_table, sin_table [N, head_dim] fp32, indexed by the token's position inside its sample. */
int sana_rope(void* x, int64_t ld, const float* cos_table, const float* sin_table, int64_t B, int64_t N, int64_t C,
              int64_t head_dim, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * ReLU linear attention, state reduction:
 *   state[b, h, i, j] = sum_n v1[b, n, h, i] * relu(k[b, n, h, j]),  v1 = [v ; 1]
 * i in [0, 33), j in [0, 32): 32 value rows plus the "ones" row that upstream creates with
 * F.pad(v, (0,0,0,1), value=1).  Replaces `vk = torch.matmul(v_pad, relu(k))` (and the
 * .float() casts before it), LiteLA.attn_matmul, diffusion/model/nets/sana_blocks.py:246-256.
 *   k, v   [B*N, *] rows of H*32 contiguous channels (head-major), row stride ld elements
 *   state  [B, H, 33, 32] fp32
 *   workspace: sana_la_state_workspace_bytes(B, N, H) bytes, 256-byte aligned; holds
 *   per-chunk partial states that a second launch adds in a fixed order (bit-reproducible).
 * Head dimension is fixed at 32 (upstream linear_head_dim).  Accumulation is fp32.
 */
int64_t sana_la_state_workspace_bytes(int64_t B, int64_t N, int64_t H);
int sana_la_state(const void* k, const void* v, int64_t ld, float* state, void* workspace,
                  int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * sana_la_state for hosts that cannot allocate device memory.  No counterpart upstream: it
 * exists for callers that may not call cudaMalloc where they run the block - a serving
 * process whose device memory is a fixed arena owned by another runtime, a plugin sandbox
 * without allocation calls, a loop that cannot afford the implicit device synchronisation
 * of cudaMalloc/cudaFree.  Same inputs, output and arithmetic as sana_la_state, but the
 * per-chunk partial states go to a scratch array built into the library image
 * (SANA_LA_STATE_NOALLOC_MAX_BYTES of device memory on every GPU that loads the library,
 * held until the process exits) instead of a caller workspace.  The call itself allocates
 * and frees nothing.
 *  - Limit: sana_la_state_workspace_bytes(B, N, H) must not exceed
 *    SANA_LA_STATE_NOALLOC_MAX_BYTES, otherwise SANA_ERR_INVALID (use sana_la_state).
 *  - The first call on each device looks up the array's device address (one host-side query,
 *    no allocation); make that first call before starting any stream capture.
 *  - All calls on a device share the one array, and it keeps whatever the previous call
 *    left; nothing in it needs clearing because each call overwrites every element it later
 *    reads.  Two calls that overlap on the GPU (different streams, or different host threads
 *    on different streams) race on it: serialise them.
 */
#define SANA_LA_STATE_NOALLOC_MAX_BYTES (16 * 1024 * 1024)
int sana_la_state_noalloc(const void* k, const void* v, int64_t ld, float* state, int64_t B, int64_t N,
                          int64_t H, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * sana_la_state for a token range sharded over the GPUs of one node: the chunk reduction is
 * fused with the all-reduce of the per-rank partial states over peer memory (NVLink loads and
 * 4-byte flag stores; no NCCL call, no multicast).  No counterpart upstream (plain LiteLA has
 * no sequence-parallel path there); the state is a plain sum over tokens, so ranks add.
 *   k, v, ld, workspace, B, N, H, dtype: as sana_la_state, for THIS rank's tokens.
 *   state [B, H, 33, 32]: the sum over all ranks, bit-identical on every rank.
 *   peer_buffers: HOST array of `world` device pointers, entry r = rank r's exchange buffer as
 *     mapped into this process (peer / symmetric memory), each sana_la_state_sp_buffer_bytes
 *     (B, H) bytes, zero-filled once before the first step.  Layout: 256 B of arrival flags,
 *     a block counter at byte 256, a soft-error word at byte 320 (non-zero = 1 + the rank that
 *     did not arrive within the wait limit - 2 s unless changed with
 *     sana_exchange_set_wait_limit_ns; the result of that step must be discarded), two state
 *     slots from byte 1024.
 *   step: 1, 2, 3, ... the same sequence on every rank, one per call on this buffer set; or 0
 *     on every call of every rank: the kernel numbers the steps itself (a word in the buffer),
 *     which lets the launch be captured in a CUDA graph and replayed.
 * Every rank must make the matching call; a rank waits inside the kernel (bounded) for the
 * others.  Launches on different GPUs only - never emulate several ranks on one GPU.
 */
int64_t sana_la_state_sp_buffer_bytes(int64_t B, int64_t H);
int sana_la_state_sp(const void* k, const void* v, int64_t ld, float* state, void* workspace,
                     int64_t workspace_bytes, int64_t B, int64_t N, int64_t H, int dtype,
                     void* const* peer_buffers, int rank, int world, uint32_t step, void* stream);

/* ---------------------------------------------------------------------------------------
 * Conv halo rows of a row-sharded token grid over peer memory: this rank's first row of the
 * depthwise conv's input goes into the upper neighbour's `bot` slot and its last row into the
 * lower neighbour's `top` slot (remote stores), a release-store of the step number tells the
 * neighbours, and the kernel returns once their rows have arrived here (bounded wait per
 * neighbour, 2 s unless changed with sana_exchange_set_wait_limit_ns; soft-error word at byte 20
 * of the buffer: bit 0 = the upper, bit 1 = the lower neighbour did not arrive).  No
 * counterpart upstream; replaces two NCCL send/recv pairs per block.
 *   first_row / last_row: [row_bytes] device rows (may be null when that neighbour is null).
 *   mine / upper / lower: exchange buffers of this rank and of ranks -1 / +1 as mapped into this
 *     process (peer / symmetric memory; null where no neighbour shares a frame),
 *     sana_halo_exchange_buffer_bytes(row_bytes) each, zero-filled once before the first step.
 *     After the call `top` is at mine + 1024 and `bot` at mine + 1024 + row_bytes.
 *   step: as in sana_la_state_sp (1, 2, 3, ... on every rank, or 0 everywhere for graph replay).
 * One slot per side suffices because every block runs a sana_la_state_sp exchange between two
 * halo exchanges.  Launches on different GPUs only.
 */
int64_t sana_halo_exchange_buffer_bytes(int64_t row_bytes);
int sana_halo_exchange(const void* first_row, const void* last_row, int64_t row_bytes, void* mine, void* upper,
                       void* lower, uint32_t step, void* stream);

/* Limit of the waits for a peer GPU inside sana_la_state_sp and sana_halo_exchange, in
 * nanoseconds (process-wide, read at launch; 0 restores the default of 2 s).  A wait that runs
 * out records its code in the buffer's soft-error word and the kernel returns; the step's result
 * must then be discarded.  No counterpart upstream (NCCL's own watchdog plays this role there). */
int sana_exchange_set_wait_limit_ns(int64_t ns);

/* ---------------------------------------------------------------------------------------
 * ReLU linear attention, apply + normalise:
 *   o[b, n, h, i] = (sum_j state[b,h,i,j] relu(q[b,n,h,j])) / (sum_j state[b,h,32,j] relu(q[b,n,h,j]) + eps)
 * Replaces `out = torch.matmul(vk, relu(q)); out[:, :, :-1] / (out[:, :, -1:] + eps)` and the
 * cast back to the model dtype, sana_blocks.py:257-263,286, written token-major so that no
 * transpose precedes the output projection (sana_blocks.py:288-289).
 *   q [B*N, *] (row stride ldq), out [B*N, *] (row stride ldo), both of `dtype`.
 */
int sana_la_apply(const void* q, int64_t ldq, const float* state, void* out, int64_t ldo, int64_t B,
                  int64_t N, int64_t H, float eps, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * ReLU linear attention with the rotation AFTER the feature map (self-attention of Sana-Video),
 * for heads of D channels, D a multiple of 16 in [16, 128] (upstream's 2B video model: 112):
 *   rot(x)[n, 2p]   = x[n, 2p] cos[n, p] - x[n, 2p+1] sin[n, p]
 *   rot(x)[n, 2p+1] = x[n, 2p] sin[n, p] + x[n, 2p+1] cos[n, p]          (channel pairs of a head)
 *   state[b, h, i, j] = sum_n v[b,n,h,i] rot(relu(k))[b,n,h,j]  (i < D);  state[b, h, D, j] = sum_n relu(k[b,n,h,j])
 *   o[b, n, h, i] = (sum_j state[b,h,i,j] rot(relu(q))[b,n,h,j]) / (sum_j state[b,h,D,j] relu(q[b,n,h,j]) + eps)
 * Replaces, in LiteLAReLURope.forward (diffusion/model/nets/sana_blocks.py:339-388), the ReLU
 * (:355-357), the complex multiplication by `rotary_emb` of q and k (:359-365), `vk = v @ k_rotated^T`
 * (:382), `z = 1 / (k.sum(-1)^T @ q + eps)` with the UNROTATED q and k (:380), `out = vk @ q_rotated`
 * (:383) and `out * z` with the cast back to the model dtype (:385), written token-major so that no
 * transpose precedes the output projection (:387-388).
 *   k, v, q, out [B*N, *] rows of H*D contiguous channels (head-major), row strides in elements
 *   cos_table, sin_table [N, D/2] fp32: real and imaginary part of upstream's complex128
 *     `rotary_emb[0, 0]` (WanRotaryPosEmbed.forward, sana_blocks.py:1393-1410), indexed by the
 *     token's position inside its sample
 *   state [B, H, D+1, D] fp32; workspace: sana_la_rope_state_workspace_bytes(B, N, H, D) bytes,
 *     16-byte aligned, holds per-chunk partial states added in a fixed order (bit-reproducible).
 * bf16: both products are tcgen05.mma instructions accumulating in tensor memory (fp32); the rotated
 * q and k are rounded to bf16 (as upstream's `type_as`) and the state enters the second product
 * rounded to bf16 (as upstream's bf16 `vk`); the key sum and the normaliser are computed in fp32.
 * fp32: plain fp32 arithmetic.
 */
int64_t sana_la_rope_state_workspace_bytes(int64_t B, int64_t N, int64_t H, int64_t D);
int sana_la_rope_state(const void* k, const void* v, int64_t ld, const float* cos_table, const float* sin_table,
                       float* state, void* workspace, int64_t workspace_bytes, int64_t B, int64_t N, int64_t H,
                       int64_t D, int dtype, void* stream);
/* The same state on top of one carried over from earlier token chunks: state = prior + (this call's sum); `prior`
 * may be `state` itself.  Replaces `cumsum_vk += _vk; cumsum_k_sum += _k.sum(...)` of ChunkCausalAttention.forward
 * (sana_blocks.py:486-488) and `vk = vk + cusum_vk; k_sum = k_sum + cumsum_k_sum` of CachedCausalAttention.forward
 * (sana_blocks.py:551-554).  sana_add_f32: out = a + b on n fp32 values (combining two such states). */
int sana_la_rope_state_add(const void* k, const void* v, int64_t ld, const float* cos_table, const float* sin_table,
                           const float* prior, float* state, void* workspace, int64_t workspace_bytes, int64_t B,
                           int64_t N, int64_t H, int64_t D, int dtype, void* stream);
int sana_add_f32(const float* a, const float* b, float* out, int64_t n, void* stream);
/* sana_la_rope_state for a token range sharded over the GPUs of one node: like sana_la_state_sp, the chunk
 * reduction does the all-reduce of the ranks' partial states over peer memory (same buffer layout, flags, step
 * numbering, wait limit and soft-error word at byte 320; exchange buffers of
 * sana_la_rope_state_sp_buffer_bytes(B, H, D) bytes, zero-filled once).  cos_table / sin_table hold the rows of
 * THIS rank's tokens.  No counterpart upstream (its sequence-parallel video attention gathers the tokens instead:
 * diffusion/distributed/context_parallel); the state is a plain sum over tokens, so ranks add.  Launches on
 * different GPUs only. */
int64_t sana_la_rope_state_sp_buffer_bytes(int64_t B, int64_t H, int64_t D);
int sana_la_rope_state_sp(const void* k, const void* v, int64_t ld, const float* cos_table, const float* sin_table,
                          float* state, void* workspace, int64_t workspace_bytes, int64_t B, int64_t N, int64_t H,
                          int64_t D, int dtype, void* const* peer_buffers, int rank, int world, uint32_t step,
                          void* stream);
int sana_la_rope_apply(const void* q, int64_t ldq, const float* cos_table, const float* sin_table,
                       const float* state, void* out, int64_t ldo, int64_t B, int64_t N, int64_t H, int64_t D,
                       float eps, int dtype, void* stream);
/* Soft-error word of the bf16 sana_la_rope_state kernel, whose tensor-core waits are bounded: 0 when
 * no wait has timed out on the current device since the last call (host-synchronising: for tests and
 * after a failure, not per step). */
int sana_la_rope_take_device_status(int* status_out);

/* ---------------------------------------------------------------------------------------
 * 3x3 depthwise conv + bias + SiLU-GLU on channels-last rows:
 *   w[y, x, c]  = b[c] + sum_{dy,dx} K[c, dy, dx] * u[y+dy-1, x+dx-1, c]   (zero outside a frame)
 *   out[y, x, c] = w[y, x, c] * silu(w[y, x, hid + c]),  c in [0, hid)
 * Replaces `depth_conv` -> `chunk(2, dim=1)` -> `glu_act` -> `a * g`,
 * GLUMBConv._apply_spatial, diffusion/model/nets/basic_modules.py:164-167 (per image, or
 * per frame when HW has three entries, :187-195).
 *   u        [rows, W, 2*hid]  local image rows; global row index = row0 + local row; a frame
 *            is H consecutive global rows (rows of different frames never mix)
 *   halo_top [W, 2*hid] = global row row0-1, halo_bot = global row row0+rows; either may be
 *            NULL when that row lies in another frame (or for a single-GPU call with
 *            row0 % H == 0 and (row0+rows) % H == 0)
 *   weight   [2*hid, 3, 3] (upstream's [2*hid, 1, 3, 3]), bias [2*hid] or NULL
 *   out      [rows, W, hid]
 * hid must be a multiple of 8.  fp32 accumulation, one rounding on store.
 */
int sana_dwconv_glu(const void* u, const void* halo_top, const void* halo_bot, const void* weight,
                    const void* bias, void* out, int64_t rows, int64_t W, int64_t H, int64_t row0,
                    int64_t hid, int dtype, void* stream);

/* Soft-error word of the bf16 sana_dwconv_glu kernel: a wait for an input row (a bulk-tensor
 * copy into shared memory) that runs out records 1 here and the warp gives up instead of
 * spinning forever.  Returns 0 when no wait timed out on the current device since the last
 * call (host-synchronising: for tests / after a failure, not per step). */
int sana_dwconv_glu_take_device_status(int* status_out);

/* ---------------------------------------------------------------------------------------
 * Softmax core of the cross-attention (image tokens over text tokens):
 *   out[b, n, h, :] = softmax_j(q[b,n,h,:] . k[b,j,h,:] / sqrt(head_dim) + (1 - mask[b,j]) * -10000) v[b,j,h,:]
 * Replaces `F.scaled_dot_product_attention(q, k, v, attn_mask=...)` and the transposes around
 * it, MultiHeadCrossAttention.forward, diffusion/model/nets/sana_blocks.py:86-93 (the 2-D mask
 * becomes the additive -10000 bias of :88-90).
 *   q   [B*N, *] row stride ldq, head h at columns h*head_dim ..   (token-major, no transposes)
 *   k,v [B*L, *] row stride ldkv (e.g. the two column blocks of the kv projection)
 *   mask [B, L] of 0/1 in the activation dtype, or NULL;  out [B*N, *] row stride ldo
 * head_dim a multiple of 8, at most 128.  bf16 with 17 <= L <= 304 and head_dim >= 16: persistent
 * tcgen05 kernel - both products on the 5th-generation tensor cores with the scores and the
 * probabilities in tensor memory, fp32 softmax in the exp2 domain, K / V of a (sample, head)
 * resident in shared memory; other bf16 shapes: warp-level tensor cores with an online softmax.
 * fp32: plain FMA (parity path).
 */
int sana_cross_attention(const void* q, int64_t ldq, const void* k, const void* v, int64_t ldkv,
                         const void* mask, void* out, int64_t ldo, int64_t B, int64_t N, int64_t L,
                         int64_t heads, int64_t head_dim, int dtype, void* stream);
/* Kernel choice of the bf16 sana_cross_attention (process-wide; for tests and measurements):
 * 0 = per problem (default), 1 = always the warp-level kernel, 2 = the tcgen05 kernel (shapes it
 * does not cover are then refused). */
int sana_cross_attention_set_variant(int variant);
/* Soft-error word of the tcgen05 cross-attention kernel, whose waits are bounded: 0 when no wait
 * has timed out on the current device since the last call (host-synchronising). */
int sana_cross_attention_take_device_status(int* status_out);

/* ---------------------------------------------------------------------------------------
 * Dense projection with fused epilogue:  out = epilogue(A @ Wt^T)
 *   A   [M, K] row stride lda;  Wt [N, K] row stride ldw (torch Linear / 1x1 Conv2d weight
 *   layout);  out [M, N] row stride ldo.
 * Epilogue, in this order, all in fp32 with one rounding on store:
 *   v = acc;  v += bias[n];  act;  v *= gate_b[n];  v += residual[m, n]
 *   act: 0 none, 1 SiLU, 2 ReLU on columns n < relu_cols, 3 GELU (tanh form)
 *   gate_b[n] = gate_table[gate_row, n] + gate_t[m / rows_per_batch, gate_row*N + n]
 * Replaces self.qkv / self.proj (sana_blocks.py:268,289), q_linear / kv_linear / proj of the
 * cross-attention (sana_blocks.py:74-75,95), inverted_conv (+ in-place SiLU) and point_conv
 * (basic_modules.py:163,167), and the gate-multiply + residual adds of
 * SanaMSBlock.forward (sana_multi_scale.py:151-155).
 * bf16: TMA-fed tcgen05 kernel, fp32 accumulation in tensor memory; requires 16-byte aligned
 * base pointers and lda, ldw, ldo, ldr multiples of 8.  f32: SIMT kernel (parity path).
 */
typedef struct sana_gemm_epilogue {
  const void* bias;       /* [N] or NULL */
  int32_t act;            /* 0 none, 1 SiLU, 2 ReLU on columns < relu_cols, 3 GELU (tanh form) */
  int32_t gate_row;       /* row of the [6, N] table (2 = gate_msa, 5 = gate_mlp) */
  int64_t relu_cols;
  const void* gate_table; /* [6, N] or NULL */
  const void* gate_t;     /* [B, 6*N]; required when gate_table != NULL */
  int64_t rows_per_batch; /* tokens per batch element (row m belongs to b = m / rows_per_batch) */
  const void* residual;   /* [M, N] row stride ldr, or NULL */
  int64_t ldr;
} sana_gemm_epilogue;

int sana_gemm(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
              int64_t N, int64_t K, const sana_gemm_epilogue* ep, int dtype, void* stream);

/* Same contract as sana_gemm but always the SIMT kernel (any dtype).  Not used by the
 * modules for bf16; it exists so tests can cross-check the tensor-core kernel on the device. */
int sana_gemm_simt(const void* A, int64_t lda, const void* Wt, int64_t ldw, void* out, int64_t ldo, int64_t M,
                   int64_t N, int64_t K, const sana_gemm_epilogue* ep, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * NVFP4 (block-scaled 4-bit) projections.  Upstream has no FP4 arithmetic of its own (it
 * wraps nn.Linear in Transformer Engine's te.Linear under an NVFP4 recipe,
 * inference_video_scripts/wm/inference_sana_wm.py:388-406); these entry points replace the
 * same nn.Linear / 1x1 Conv2d calls as sana_gemm with both operands quantised.
 *
 * Format: E2M1 values {0, .5, 1, 1.5, 2, 3, 4, 6} with sign, two per byte (even K index in
 * the low nibble), one E4M3 scale per 16 consecutive K elements, one fp32 scale per tensor:
 *   x ~ code * block_scale * tensor_scale,  tensor_scale = amax / (6 * 448),
 *   block_scale = E4M3(block_amax * (1 / (6 * tensor_scale))),
 *   code = E2M1(x * (1 / (block_scale * tensor_scale)))
 * (reciprocals and products in fp32; every step rounds to nearest even, conversions saturate).  Block scales are stored in 512-byte tiles of
 * 128 rows x 4 blocks, byte (r % 32) * 16 + (r / 32) * 4 + b, tiles K-fastest with the K-tile
 * count padded to a multiple of 4 (sana_nvfp4_sf_bytes gives the buffer size).
 *
 * sana_nvfp4_quantize: x [rows, K] bf16 (row stride ld) -> q [rows, K/2] bytes, sf (scale
 *   tiles), scales[2] = {amax, tensor_scale} (device floats).  K % 32 == 0.  Three launches:
 *   absolute maximum, then quantise; nothing is read back to the host.
 * sana_gemm_nvfp4: out[M, N] bf16 = epilogue(a_scales[1] * w_scales[1] * Aq @ Wq^T) with the
 *   sana_gemm epilogue.  tcgen05.mma kind::mxf4nvf4 (block 16) with scales in tensor memory;
 *   M >= 2048: CTA pairs (cta_group::2) on 256 x 256 tiles, else one CTA on 128 x 128 tiles
 *   (sana_gemm_set_variant overrides the choice).
 */
int64_t sana_nvfp4_sf_bytes(int64_t rows, int64_t K);
int sana_nvfp4_quantize(const void* x, int64_t ld, void* q, void* sf, float* scales, int64_t rows, int64_t K,
                        void* stream);
int sana_gemm_nvfp4(const void* Aq, const void* sfa, const float* a_scales, const void* Wq, const void* sfw,
                    const float* w_scales, void* out, int64_t ldo, int64_t M, int64_t N, int64_t K,
                    const sana_gemm_epilogue* ep, void* stream);
int sana_gemm_nvfp4_take_device_status(int* status_out);

/* ---------------------------------------------------------------------------------------
 * Activations quantised where they are produced ("delayed scaling").  Upstream leaves the
 * quantisation of a projection's input to Transformer Engine's te.Linear
 * (inference_video_scripts/wm/inference_sana_wm.py:388-406), which measures the tensor's maximum
 * and quantises in passes of its own; the exact per-tensor maximum of a tensor cannot be known
 * while it is still being produced.  Here the producing kernel writes E2M1 codes and E4M3 block
 * scales directly, with the per-tensor scale taken from a record that an EARLIER call has
 * filled, and notes the largest magnitude it produces for the calls that follow:
 *   state  n records of four device floats {amax in use, tensor scale in use, amax seen since
 *          the last roll, unused}.  sana_nvfp4_scale_roll adopts "seen" x margin as the values
 *          in use (records that saw nothing keep theirs).  A record doubles as the `scales`
 *          argument of sana_gemm_nvfp4.  Values above the amax in use saturate, so the first
 *          call on new data should be a measured one (sana_nvfp4_quantize) whose amax is copied
 *          into the record.
 *   scale_in = record (uses scale_in[1]);  amax_out = record + 2 (may be NULL).
 * With the same amax the codes and block scales equal those of sana_nvfp4_quantize applied to
 * the bf16 tensor bit for bit (the value is rounded to bf16 before it is quantised).
 *   sana_ln_modulate_fp4   sana_ln_modulate (bf16) whose output goes to q / sf (K = C); z may be
 *                          NULL (no bf16 copy).  C % 32 == 0.
 *   sana_la_apply_fp4      sana_la_apply (bf16) whose output goes to fq / sf (K = H * 32); out may
 *                          be NULL.
 *   sana_dwconv_glu_amax   sana_dwconv_glu (bf16) that also raises *amax_out to max |out|.
 *   sana_nvfp4_quantize_scaled   sana_nvfp4_quantize without the measuring pass: scales[0] holds
 *                          the amax to scale for.
 * sf buffers must be zero-filled once by their owner (bytes of padding rows / tiles are never
 * written). */
int sana_nvfp4_scale_roll(float* state, int64_t n, float margin, void* stream);
int sana_nvfp4_quantize_scaled(const void* x, int64_t ld, void* q, void* sf, float* scales, int64_t rows, int64_t K,
                               void* stream);
int sana_ln_modulate_fp4(const void* x, const void* table, const void* t, void* z, void* q, void* sf,
                         const float* scale_in, float* amax_out, int64_t B, int64_t N, int64_t C, int shift_row,
                         int scale_row, float eps, void* stream);
int sana_la_apply_fp4(const void* q, int64_t ldq, const float* state, void* out, int64_t ldo, void* fq, void* sf,
                      const float* scale_in, float* amax_out, int64_t B, int64_t N, int64_t H, float eps, void* stream);
int sana_dwconv_glu_amax(const void* u, const void* halo_top, const void* halo_bot, const void* weight,
                         const void* bias, void* out, int64_t rows, int64_t W, int64_t H, int64_t row0,
                         int64_t hid, float* amax_out, void* stream);

/* Soft-error word of the tensor-core GEMM: its bounded waits record a code here instead of
 * spinning forever.  Returns 0 when no wait ever timed out on the current device since the
 * last call (host-synchronising: use in tests / after a failure, not per step). */
int sana_gemm_take_device_status(int* status_out);

/* Kernel choice of the bf16 sana_gemm (process-wide; for tests and measurements):
 * 0 = per problem (default: CTA-pair kernel, tcgen05 cta_group::2 with 256-row tiles, when
 * M >= 2048, else the single-CTA kernel), 1 = always single-CTA, 2 = always CTA-pair. */
int sana_gemm_set_variant(int variant);

/* ---------------------------------------------------------------------------------------
 * Steps either side of the block loop of `SanaMS.forward`
 * (diffusion/model/nets/sana_multi_scale.py:338-386).
 *
 * sana_patchify: latent x [B, Cin, H, W] -> rows [B*(H/p)*(W/p), Cin*p*p] (row stride ldo),
 *   column (c*p + i)*p + j = x[b, c, hp*p + i, wp*p + j].  With the conv weight
 *   [embed, Cin, p, p] viewed as [embed, Cin*p*p], sana_gemm on these rows is
 *   `PatchEmbedMS.forward` (sana_blocks.py:1263-1268: Conv2d kernel = stride = p, flatten(2),
 *   transpose(1, 2)); the sin-cos position table goes in as the GEMM's residual.
 * sana_unpatchify: tokens [B*Hp*Wp, p*p*Cout] (row stride ld) -> images [B, Cout, Hp*p, Wp*p];
 *   replaces `SanaMS.unpatchify` (sana_multi_scale.py:409-421, einsum "nhwpqc->nchpwq").
 * sana_timestep_embedding: t [B] fp32 -> out [B, dim] of `dtype`, cos | sin halves with
 *   frequencies exp(-ln(max_period) k / (dim/2)); replaces
 *   `TimestepEmbedder.timestep_embedding` (sana_blocks.py:981-1000).
 * sana_silu: out = x * sigmoid(x) on n elements; the `nn.SiLU()` in front of `t_block`'s
 *   linear (sana_multi_scale.py:241), whose input is also needed without the activation.
 */
int sana_patchify(const void* x, void* out, int64_t ldo, int64_t B, int64_t Cin, int64_t H, int64_t W, int64_t p,
                  int dtype, void* stream);
int sana_unpatchify(const void* tok, int64_t ld, void* out, int64_t B, int64_t Cout, int64_t Hp, int64_t Wp, int64_t p,
                    int dtype, void* stream);
int sana_timestep_embedding(const float* t, void* out, int64_t B, int64_t dim, float max_period, int dtype,
                            void* stream);
int sana_silu(const void* x, void* out, int64_t n, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SANA_B200_H_ */
