/* C ABI of the B200-native Pairformer hot-path library (libof3b200.so).
 *
 * Plain C: raw device pointers, explicit shapes, a cudaStream_t passed as void*. No torch
 * or C++ types cross this boundary. All "reference" citations are paths inside the
 * aqlaboratory/openfold-3 source tree.
 *
 * Conventions
 *  - Return value: 0 ok; < 0 argument / shape / alignment / workspace error (OF3_ERR_*);
 *    > 0 a cudaError_t. of3_last_error_string() describes the last failure of the calling
 *    thread. Nothing throws or aborts.
 *  - dtype: OF3_DTYPE_BF16 (bf16 storage, fp32 accumulation and statistics) or
 *    OF3_DTYPE_F32 (fp32 storage and true fp32 arithmetic: the validation mode). Activations,
 *    masks and parameters of one call share the dtype.
 *  - Every buffer is owned by the caller. Entry points enqueue work on `stream` and return;
 *    they allocate nothing (except a 64-byte per-device status block on first use) and keep
 *    no reference after the enqueued work completes. `workspace` must hold at least the
 *    matching *_workspace_bytes() and stay valid until the stream reaches the end of the call.
 *  - `out` may alias the input activation (in-place residual update) where noted.
 *  - flags: OF3_FLAG_ADD_RESIDUAL writes input + update instead of the update;
 *    OF3_FLAG_FORCE_GENERIC selects the shape-generic SIMT kernels even where a tcgen05
 *    kernel exists (used by tests to cross-check the two families).
 *  - Thread safety: re-entrant; calls are ordered by the stream they are given.
 */
#ifndef OF3B200_H
#define OF3B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OF3_OK 0
#define OF3_ERR_ARG (-1)
#define OF3_ERR_SHAPE (-2)
#define OF3_ERR_ALIGN (-3)
#define OF3_ERR_WORKSPACE (-4)
#define OF3_ERR_DRIVER (-5)
#define OF3_ERR_DEVICE_WAIT (-6)

#define OF3_DTYPE_BF16 0
#define OF3_DTYPE_F32 1

#define OF3_FLAG_ADD_RESIDUAL 1
#define OF3_FLAG_FORCE_GENERIC 2
#define OF3_FLAG_OUTGOING 4    /* trimul: outgoing edges (else incoming) */
#define OF3_FLAG_TRANSPOSED 8  /* triangle attention around the ending node */
#define OF3_FLAG_ADA_LN 16     /* attention pair bias: adaptive LayerNorm conditioning on s */

/* Message for the last non-zero return code seen by the calling thread. */
const char* of3_last_error_string(void);

/* Device-side status block: kernels with bounded waits (mbarrier / TMEM pipelines) record
 * {code, kernel id, block, wait site} here instead of spinning forever. Synchronises the device. */
int of3_device_status(int* out4);
int of3_device_status_clear(void);
/* Stream-ordered copy of the four status words into pinned host memory; no synchronisation. */
int of3_device_status_async(int* host4, void* stream);

/* Launch accounting. Every kernel launch of the library is counted per kernel id; with timing
 * enabled a CUDA-event pair is recorded around each launch on the launching stream (the events
 * come from a pool that grows on demand). of3_profile_read synchronises the device and returns the
 * launches since the last reset and the summed device time of the timed ones.
 * Kernel ids: 1 triangle contraction, 2 trimul projection/gate, 3 trimul output, 4 SwiGLU
 * transition, 5 attention projection, 6 attention core, 7 attention output, 20 generic kernels. */
int of3_profile_enable(int on);
int of3_profile_reset(void);
int of3_profile_read(int kernel_id, long long* launches, float* total_ms);

/* 1 when the tcgen05 kernel family covers this shape and dtype, else 0 (generic kernels run). */
int of3_fast_path_available(int module_id, int dtype, int c, int c_hidden, int heads, int head_dim);
#define OF3_MODULE_TRIMUL 1
#define OF3_MODULE_TRIATTN 2
#define OF3_MODULE_TRANSITION 3

/* ---- Triangle multiplicative update ------------------------------------------------------
 * Replaces TriangleMultiplicativeUpdate.forward / _inference_forward
 * (openfold3/core/model/layers/triangular_multiplicative_update.py:421-503, 154-419) and the
 * operator seam _cueq_triangle_mult (:689-741).
 * z, out: [B, N, N, c_z]; mask: [B, N, N] or NULL (all ones). out may alias z. */
typedef struct {
    const void* ln_in_w;   /* [c_z] layer_norm_in.weight */
    const void* ln_in_b;   /* [c_z] layer_norm_in.bias */
    const void* w_a_p;     /* [c_h, c_z] linear_a_p.weight */
    const void* w_a_g;     /* [c_h, c_z] linear_a_g.weight */
    const void* w_b_p;     /* [c_h, c_z] linear_b_p.weight */
    const void* w_b_g;     /* [c_h, c_z] linear_b_g.weight */
    const void* w_g;       /* [c_z, c_z] linear_g.weight */
    const void* ln_out_w;  /* [c_h] layer_norm_out.weight */
    const void* ln_out_b;  /* [c_h] layer_norm_out.bias */
    const void* w_z;       /* [c_z, c_h] linear_z.weight */
} of3_trimul_params;

size_t of3_trimul_workspace_bytes(int B, int N, int c_z, int c_h, int dtype, int flags);
int of3_trimul_forward(const void* z, const void* mask, void* out, int B, int N, int c_z, int c_h,
                       int dtype, int flags, const of3_trimul_params* p, void* workspace,
                       size_t workspace_bytes, void* stream);

/* Triangle multiplicative update for callers that cannot allocate device memory (a process with a
 * frozen memory budget, a plugin running inside another component's stream-ordered region, an
 * embedder that only forwards the tensors it was given). No counterpart in the reference: its
 * modules always allocate their temporaries through PyTorch.
 * Same arguments and semantics as of3_trimul_forward minus the workspace: the intermediates live
 * in a 16 MiB array built into the library (held by every GPU that loads it, until exit). It runs
 * the shape-generic kernels and calls no cudaMalloc / cudaFree or allocating library routine.
 *  - Limit: B*N*N*max(c_z, c_h)*24 bytes must fit in of3_trimul_static_scratch_bytes()
 *    (N <= 73 at B = 1, c = 128); beyond it the call returns OF3_ERR_WORKSPACE.
 *  - The first call on a device resolves the array's device address; make it before any stream
 *    capture.
 *  - Every call uses the same array, which keeps the previous call's contents (none of it needs
 *    to start at zero). Calls that overlap on the GPU race on it: keep them ordered. */
size_t of3_trimul_static_scratch_bytes(void);
int of3_trimul_forward_static(const void* z, const void* mask, void* out, int B, int N, int c_z, int c_h,
                              int dtype, int flags, const of3_trimul_params* p, void* stream);

/* ---- Triangle attention ------------------------------------------------------------------
 * Replaces TriangleAttention.forward (openfold3/core/model/layers/triangular_attention.py:
 * 102-167) including the gated multi-head attention it calls
 * (openfold3/core/model/primitives/attention.py:346-413, _attention :94-135) and the operator
 * seams _cueq_triangle_attn (:625-672) / _deepspeed_evo_attn (:489-560).
 * With OF3_FLAG_TRANSPOSED the layer acts on z^T and mask^T and the update is transposed back,
 * which is both TriangleAttentionEndingNode and what PairBlock.tri_att_start_end does around
 * tri_att_end (openfold3/core/model/latent/base_blocks.py:380-404) -- without moving z.
 * z, out: [B, N, N, c_z]; mask: [B, N, N] or NULL. out may alias z. inf: the mask constant. */
typedef struct {
    const void* ln_w;    /* [c_z] layer_norm.weight */
    const void* ln_b;    /* [c_z] layer_norm.bias */
    const void* w_bias;  /* [H, c_z] linear_z.weight (triangle bias) */
    const void* w_q;     /* [H*d, c_z] mha.linear_q.weight */
    const void* w_k;     /* [H*d, c_z] mha.linear_k.weight */
    const void* w_v;     /* [H*d, c_z] mha.linear_v.weight */
    const void* w_g;     /* [H*d, c_z] mha.linear_g.weight */
    const void* w_o;     /* [c_z, H*d] mha.linear_o.weight */
} of3_triattn_params;

size_t of3_triattn_workspace_bytes(int B, int N, int c_z, int H, int d, int dtype, int flags);
int of3_triattn_forward(const void* z, const void* mask, void* out, int B, int N, int c_z, int H,
                        int d, float inf, int dtype, int flags, const of3_triattn_params* p,
                        void* workspace, size_t workspace_bytes, void* stream);

/* ---- SwiGLU transition -------------------------------------------------------------------
 * Replaces SwiGLUTransition (openfold3/core/model/layers/transition.py:225-271) with its
 * SwiGLU (openfold3/core/model/primitives/activations.py:33-61), for the pair (c=128) and the
 * single (c=384) track. x, out: [rows, c]; mask: [rows] or NULL; hidden width n*c.
 * out may alias x. */
typedef struct {
    const void* ln_w;   /* [c] layer_norm.weight */
    const void* ln_b;   /* [c] layer_norm.bias */
    const void* w_a;    /* [n*c, c] swiglu.linear_a.weight */
    const void* w_b;    /* [n*c, c] swiglu.linear_b.weight */
    const void* w_out;  /* [c, n*c] linear_out.weight */
} of3_transition_params;

size_t of3_transition_workspace_bytes(long long rows, int c, int n, int dtype, int flags);
int of3_transition_forward(const void* x, const void* mask, void* out, long long rows, int c, int n,
                           int dtype, int flags, const of3_transition_params* p, void* workspace,
                           size_t workspace_bytes, void* stream);

/* ---- Attention with pair bias ------------------------------------------------------------
 * Replaces AttentionPairBias.forward (openfold3/core/model/layers/attention_pair_bias.py:
 * 123-227) for the trunk single track (LayerNorm) and, with OF3_FLAG_ADA_LN, for the diffusion
 * token track (AdaLN, openfold3/core/model/primitives/normalization.py:89-140).
 * a, out: [Ba, N, c_a]; z: [Bz, N, N, c_z] with Ba a multiple of Bz (samples sharing one pair
 * tensor are consecutive); s: [Ba, N, c_s] (AdaLN only, else NULL); mask: [Ba, N] or NULL.
 * out may alias a.
 * Launch grouping (bf16 kernels; an optimisation, never a requirement): linear layers that read the
 * same input run as ONE launch when their weights lie back to back in memory -- here w_q, w_g, w_k,
 * w_v in this order (w_g == w_q + H*d*c_a elements, ...) and ada_w_g, ada_w_s; in
 * of3_cond_transition_params ada_w_g, ada_w_s and w_a, w_b; in of3_transition_params w_a, w_b.
 * Otherwise each layer is its own launch, with the same result. */
typedef struct {
    const void* ln_a_w;      /* [c_a] layer_norm_a.weight              (LayerNorm variant) */
    const void* ln_a_b;      /* [c_a] layer_norm_a.bias                (LayerNorm variant) */
    const void* ada_ln_s_w;  /* [c_s] layer_norm_a.layer_norm_s.weight (AdaLN variant) */
    const void* ada_w_g;     /* [c_a, c_s] layer_norm_a.linear_g.weight */
    const void* ada_b_g;     /* [c_a] layer_norm_a.linear_g.bias */
    const void* ada_w_s;     /* [c_a, c_s] layer_norm_a.linear_s.weight */
    const void* w_ada_out;   /* [c_a, c_s] linear_ada_out.weight       (AdaLN variant) */
    const void* b_ada_out;   /* [c_a] linear_ada_out.bias */
    const void* ln_z_w;      /* [c_z] layer_norm_z.weight */
    const void* ln_z_b;      /* [c_z] layer_norm_z.bias or NULL */
    const void* w_z;         /* [H, c_z] linear_z.weight */
    const void* w_q;         /* [H*d, c_a] mha.linear_q.weight */
    const void* b_q;         /* [H*d] mha.linear_q.bias or NULL */
    const void* w_k;         /* [H*d, c_a] */
    const void* w_v;         /* [H*d, c_a] */
    const void* w_g;         /* [H*d, c_a] */
    const void* w_o;         /* [c_a, H*d] */
} of3_attn_pair_bias_params;

size_t of3_attn_pair_bias_workspace_bytes(int Ba, int Bz, int N, int c_a, int c_s, int c_z, int H,
                                          int d, int dtype, int flags);
int of3_attn_pair_bias_forward(const void* a, const void* z, const void* s, const void* mask,
                               void* out, int Ba, int Bz, int N, int c_a, int c_s, int c_z, int H,
                               int d, float inf, int dtype, int flags,
                               const of3_attn_pair_bias_params* p, void* workspace,
                               size_t workspace_bytes, void* stream);

/* ---- Conditioned (AdaLN) SwiGLU transition -----------------------------------------------
 * Replaces ConditionedTransitionBlock (openfold3/core/model/layers/transition.py:274-380).
 * a, out: [rows, c_a]; s: [rows, c_s]; mask: [rows] or NULL. out may alias a. */
typedef struct {
    const void* ada_ln_s_w;  /* [c_s] layer_norm.layer_norm_s.weight */
    const void* ada_w_g;     /* [c_a, c_s] layer_norm.linear_g.weight */
    const void* ada_b_g;     /* [c_a] layer_norm.linear_g.bias */
    const void* ada_w_s;     /* [c_a, c_s] layer_norm.linear_s.weight */
    const void* w_a;         /* [n*c_a, c_a] swiglu.linear_a.weight */
    const void* w_b;         /* [n*c_a, c_a] swiglu.linear_b.weight */
    const void* w_g;         /* [c_a, c_s] linear_g.weight */
    const void* b_g;         /* [c_a] linear_g.bias */
    const void* w_out;       /* [c_a, n*c_a] linear_out.weight */
} of3_cond_transition_params;

size_t of3_cond_transition_workspace_bytes(long long rows, int c_a, int c_s, int n, int dtype,
                                           int flags);
int of3_cond_transition_forward(const void* a, const void* s, const void* mask, void* out,
                                long long rows, int c_a, int c_s, int n, int dtype, int flags,
                                const of3_cond_transition_params* p, void* workspace,
                                size_t workspace_bytes, void* stream);

/* ---- Row-sharded ("DAP") pair stack: phase entry points --------------------------------------
 * No counterpart in the reference (it has data-parallel DDP / ZeRO only;
 * openfold3/entry_points/experiment_runner.py:218-246). Each of the P ranks (P = 1, 2, 4, 8) owns
 * R = N / P consecutive rows of one sample's pair tensor (bf16, c_z = c_hidden = 128, 4 heads x 32)
 * and runs every layer as phases around the exchanges the layer needs; the exchanges (all-to-all /
 * all-gather) are the caller's, between the calls. Pitches: ld(n) = of3_dap_pitch(n, 8) for the
 * triangle update's planes.
 *
 * Triangle update (triangular_multiplicative_update.py:421-503), C = 128 / P channels per rank:
 *   project   z_rows -> ab [P][2][C][lines][ld(positions)]: the gated projections a (index 0) and b
 *             (index 1), channel-major, grouped by the rank that will contract each channel.
 *             outgoing: transposed = 0, z_rows [lines = R][positions = N][128], mask [R][N];
 *             incoming: transposed = 1, the same memory read as [positions = R][lines = N][128]
 *             (a line runs along the local rows), mask [R][N] likewise.
 *   (all-to-all of the P blocks, then regroup to ab_all [2][C][N][ld(N)]: of3_copy_rows_3d)
 *   contract  x[c][i][j] = sum_k a[c][i][k] b[c][j][k] for this rank's C channels and ALL i, j, written as
 *             x_blocks [P][C][R][ld(N)]: block q holds rows q*R .. q*R + R - 1, i.e. what rank q needs
 *   (all-to-all of the P blocks: x_t [128][R][ld(N)] = this rank's rows of every channel)
 *   output    LayerNorm_out(x) -> linear_z, sigmoid(linear_g(LayerNorm_in(z))) gate, residual, on z_rows.
 * Attention: z_rows, out_rows [R, N, 128]; mask_rows [R, N] or NULL; q, k, vt: opaque images of
 *   of3_dap_triattn_image_elems(R, N) elements each (pre-swizzled operand tiles); the pair bias is a
 *   bf16 image, pre-scaled by log2(e): bias_rows [4 heads][nkb = ceil(N / 32) key blocks][R query rows][32]
 *   (of3_dap_triattn_bias_elems(R, N) elements; each 64-byte row in tensor-core operand order, which
 *   depends on the row's index among all N query rows: row0 = index of this rank's first row), bias_all the
 *   same with all N query rows [4][nkb][N][32]: an all-gather of the ranks' rows along the third index;
 *   o_scratch [R, N, 128]. out_rows may alias z_rows. */
int of3_dap_pitch(int N, int multiple);
long long of3_dap_triattn_image_elems(int R, int N);
long long of3_dap_triattn_bias_elems(int R, int N);
int of3_dap_trimul_project(const void* z_rows, const void* mask, void* ab, int lines, int positions, int transposed,
                           int world, const of3_trimul_params* p, void* stream);
int of3_dap_trimul_contract(const void* ab_all, void* x_blocks, int N, int channels, int rows_per_rank,
                            void* stream);
int of3_dap_trimul_output(const void* z_rows, void* out_rows, const void* x_t, int R, int N, int flags,
                          const of3_trimul_params* p, void* stream);
/* Strided copy of n0*n1*n2 rows of row_bytes bytes; row (i0, i1, i2) is read at src + i0*s0 + i1*s1 +
 * i2*s2 and written at dst + i0*t0 + i1*t1 + i2*t2 (byte strides). The repacks between an
 * all-to-all's rank-major blocks and the layouts the kernels read. */
int of3_copy_rows_3d(const void* src, void* dst, int n0, int n1, int n2, long long s0, long long s1, long long s2,
                     long long t0, long long t1, long long t2, int row_bytes, void* stream);
int of3_dap_triattn_project(const void* z_rows, void* q, void* k, void* vt, void* bias_rows, int R, int N, int row0,
                            const of3_triattn_params* p, void* stream);
int of3_dap_triattn_finish(const void* z_rows, const void* mask_rows, void* out_rows, const void* q, const void* k,
                           const void* vt, const void* bias_all, void* o_scratch, int R, int N, float inf, int flags,
                           const of3_triattn_params* p, void* stream);
/* Pair-bias projection of AttentionPairBias (attention_pair_bias.py:154-163) for `positions` pair
 * positions: bias_rows[h][pos] = linear_z(LayerNorm_z(z))[pos][h], fp32, c_z = 128, 16 heads. */
int of3_pair_bias_project(const void* z_rows, const void* ln_w, const void* ln_b, const void* w, float* bias_rows,
                          long long positions, int c_z, int H, int dtype, void* stream);
/* of3_attn_pair_bias_forward with the pair bias [Bz, H, N, N] (fp32) already projected. */
int of3_attn_pair_bias_forward_prebias(const void* a, const float* pair_bias, const void* s, const void* mask,
                                       void* out, int Ba, int Bz, int N, int c_a, int c_s, int H, int d, float inf,
                                       int dtype, int flags, const of3_attn_pair_bias_params* p, void* workspace,
                                       size_t workspace_bytes, void* stream);
/* The same two steps without the fp32 tensor in between (bf16 only): the projection of ONE sample's pair
 * tensor z [N, N, 128] written as the attention kernel's own bias tiles -- bf16, times log2(e),
 * [16 heads][ceil(N / 32) key blocks][N query rows][32 keys], of3_pair_bias_tiles_elems(N) elements; samples
 * of a batch lie back to back -- and the layer taking tiles [Bz][...]. A caller that applies the layer many
 * times to one pair tensor (a diffusion rollout) keeps the tiles. */
long long of3_pair_bias_tiles_elems(int N);
int of3_pair_bias_project_tiles(const void* z, const void* ln_w, const void* ln_b, const void* w, void* tiles, int N,
                                int c_z, int H, int dtype, void* stream);
int of3_attn_pair_bias_forward_pretiles(const void* a, const void* bias_tiles, const void* s, const void* mask,
                                        void* out, int Ba, int Bz, int N, int c_a, int c_s, int H, int d, float inf,
                                        int dtype, int flags, const of3_attn_pair_bias_params* p, void* workspace,
                                        size_t workspace_bytes, void* stream);

/* The AttentionPairBias layer (attention_pair_bias.py:123-227, LayerNorm variant) for a window of R
 * query rows [row0, row0 + R) of one sample: keys / values from all N rows of a [N, c_a], the pair bias
 * of exactly those rows (pair_bias_rows [H, R, N], fp32), out_rows [R, c_a]. bf16, 16 heads of 24 / 48. */
size_t of3_attn_pair_bias_rows_workspace_bytes(int N, int R, int c_a);
int of3_attn_pair_bias_forward_rows(const void* a, const float* pair_bias_rows, const void* mask, void* out_rows,
                                    int N, int row0, int R, int c_a, int H, int d, float inf, int dtype, int flags,
                                    const of3_attn_pair_bias_params* p, void* workspace, size_t workspace_bytes,
                                    void* stream);

/* ---- Exchanges over NVLink peer memory (no counterpart in the reference) --------------------
 * One "peer heap" per rank: device memory of this process that the other ranks of the node map into
 * their own address space (CUDA IPC). alloc returns the local pointer and a 64-byte handle to pass to
 * the other processes (any host transport); open maps a peer's heap; close / free undo them.
 * of3_peer_barrier: a one-warp kernel; returns (on the stream) once every rank has launched the same
 *   barrier. flag_blocks[r] = address IN THIS PROCESS of a zero-initialised 64-byte block inside rank r's
 *   heap (the same offset on every rank). Waits are bounded (2 s; 60 s for of3_peer_barrier_step_entry, the
 *   first barrier of a step, where the ranks' hosts may be far apart), then of3_device_status reports kernel
 *   30, every later of3_peer_pull_rows of the process moves nothing and later barriers do not wait, until
 *   of3_device_status_clear: a step whose barrier failed cannot produce a silently wrong result.
 * of3_peer_pull_rows: world*n1*n2 rows of row_bytes; row (r, i1, i2) is read from rank r's heap at
 *   srcs[r] + src_off + i1*s1 + i2*s2 and written to dst + r*t0 + i1*t1 + i2*t2 (byte strides):
 *   all-to-all, all-gather and the repack into the consumer's layout in one pass. Call it after a
 *   barrier that follows the producers; a buffer may be rewritten once a later barrier has passed. */
int of3_peer_heap_alloc(size_t bytes, void** ptr, void* handle64);
int of3_peer_heap_open(const void* handle64, void** ptr);
int of3_peer_heap_close(void* ptr);
int of3_peer_heap_free(void* ptr);
int of3_peer_barrier(void* const* flag_blocks, int world, int rank, void* stream);
int of3_peer_barrier_step_entry(void* const* flag_blocks, int world, int rank, void* stream);
int of3_peer_pull_rows(void* const* srcs, long long src_off, void* dst, int world, int rank, int n1, int n2,
                       long long s1, long long s2, long long t0, long long t1, long long t2, int row_bytes,
                       void* stream);
/* The same index space with the roles swapped: row (r, i1, i2) is read from the local src + r*t0 + i1*t1 +
 * i2*t2 and written into rank r's heap at dsts[r] + dst_off + i1*s1 + i2*s2. Follow it with a barrier. */
int of3_peer_push_rows(void* const* dsts, long long dst_off, const void* src, int world, int rank, int n1, int n2,
                       long long s1, long long s2, long long t0, long long t1, long long t2, int row_bytes,
                       void* stream);

/* ---- Building block exported for tests and profiling --------------------------------------
 * X[b][i][j] = sum_k A[b][i][k] * B[b][j][k], bf16 in / fp32 accumulate / bf16 out, the
 * tcgen05 kernel behind the triangle contraction (einsum of
 * triangular_multiplicative_update.py:71-97). Pitches and batch strides in elements. */
int of3_contract_nt_bf16(const void* a, const void* b, void* out, int batch, int M, int N, int K,
                         int lda, int ldb, int ldo, long long a_batch_stride,
                         long long b_batch_stride, long long out_batch_stride, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OF3B200_H */
