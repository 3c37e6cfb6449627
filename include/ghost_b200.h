/*
 * ghost_b200.h -- C ABI of libghost_b200.so: the per-sample-gradient ("ghost") layer math of
 * GhostSuite as hand-written sm_100a CUDA kernels.
 *
 * Conventions
 *   - Every function returns an int status: GHOST_OK (0) or a negative GHOST_ERR_* code;
 *     ghost_last_error() returns a thread-local message for the last failure.  Nothing aborts
 *     and nothing falls back to another implementation: an unsupported shape, dtype or GPU is an
 *     error.
 *   - All data pointers are DEVICE pointers owned by the caller (inputs, outputs, workspaces).
 *     The library never allocates device memory.  `stream` is a cudaStream_t passed as void*;
 *     work is enqueued on it and no call synchronises the device, except ghost_poll_kernel_error.
 *   - Batch layout: train samples first, validation samples last along the leading dimension
 *     (GhostSuite: ghostEngines/engine_manager.py:201-202).
 *   - Sizes are in elements, pitches ("ld") in elements of the pointed-to type.
 *   - bf16 operands that feed TMA need a 16-byte aligned base and a pitch that is a multiple of
 *     8 elements; ghost_cast_split_bf16 produces such copies from any fp32 / bf16 tensor.
 *   - Dot-product outputs are always the full matrix M[n_val, n_train] (row-major fp32);
 *     GhostSuite's grad_dot_prod vector is its column sum over the validation samples.
 *
 * "Replaces" comments cite the GhostSuite source (file:line) whose computation the entry point
 * takes over.
 */
#ifndef GHOST_B200_H_
#define GHOST_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

enum {
  GHOST_OK = 0,
  GHOST_ERR_INVALID = -1,        /* bad argument (the Python layer raises ValueError) */
  GHOST_ERR_CUDA = -2,           /* a CUDA runtime / driver call failed */
  GHOST_ERR_DEVICE = -3,         /* current device is not sm_100 */
  GHOST_ERR_KERNEL_TIMEOUT = -4, /* a kernel gave up a bounded wait (see ghost_poll_kernel_error) */
  GHOST_ERR_INDEX = -5           /* a kernel met an embedding id outside [0, vocab) (the Python layer raises IndexError) */
};

/* ---- library / device ---------------------------------------------------------------------- */
const char* ghost_version(void);
const char* ghost_last_error(void);
/* GHOST_OK iff the current CUDA device is a B200-class (sm_100) GPU. */
int ghost_device_check(void);
int ghost_sm_count(void);
/* Number of kernels this library has launched in this process (all threads, all devices). */
long long ghost_launch_count(void);
/* Reads (synchronously) the per-device word that kernels set when a bounded mbarrier wait ran out or
 * an out-of-range embedding id was met.  Returns GHOST_OK, GHOST_ERR_KERNEL_TIMEOUT or
 * GHOST_ERR_INDEX; `clear` resets the word. */
int ghost_poll_kernel_error(int clear);

/* ---- operand preparation --------------------------------------------------------------------- */
/* dst (bf16) <- src (fp32 if src_is_f32 else bf16), rows = samples * T, zero-padded to `cpad`
 * columns, written `parts` (1..3) times.  kind_i = 0 writes bf16(x); kind_i = 1 writes the residual
 * bf16(x - bf16(x)), so that fp32 inputs can be contracted on the bf16 tensor pipe with fp32-class
 * accuracy (hi*hi + lo*hi + hi*lo).  row_stack = 0: parts side by side along columns
 * (ld_dst >= parts * cpad); row_stack = 1: parts stacked along rows inside each sample, i.e. dst is
 * [samples, parts * T, cpad].
 * Replaces the .to(torch.bfloat16) casts of
 * ghostEngines/supported_layers_grad_samplers_dotprod.py:92-93, 396-397. */
int ghost_cast_split_bf16(const void* src, int src_is_f32, long long samples, long long T, int cols,
                          long long ld_src, void* dst, long long ld_dst, int cpad, int parts,
                          int kind0, int kind1, int kind2, int row_stack, void* stream);

/* ---- Linear / Conv1D weight dot product, Gram ("ghost") path --------------------------------- */
/* M[v,b] = scale * sum_{t in b, s in v} (a_train[t] . a_val[s]) * (g_train[t] . g_val[s]).
 * a_*: [n_* * T, ka] bf16, g_*: [n_* * T, kg] bf16.  round_mode 0: fp32 Gram entries multiplied in
 * fp32; round_mode 1: Gram entries and their product rounded to bf16 as GhostSuite does.
 * One fused tcgen05/TMEM kernel; the Gram matrices are never written to memory.
 * Replaces ghostEngines/supported_layers_grad_samplers_dotprod.py:119-130 (Linear) and :416-437
 * (Conv1D), per validation sample. */
int ghost_gram_dot_bf16(const void* a_train, const void* a_val, const void* g_train,
                        const void* g_val, int n_train, int n_val, long long T, int ka, int kg,
                        long long ld_at, long long ld_av, long long ld_gt, long long ld_gv,
                        int round_mode, float scale, float* M_out, void* stream);

/* Selects the kernel behind ghost_gram_dot_bf16: 0 = one CTA per 128 x 256 tile; 1 (default) = a
 * CTA pair (tcgen05 cta_group::2) per 256 x 256 tile for problems of at least 512 train tokens and
 * 256 to 8192 validation tokens; 2 = the pair kernel from 512 x 256 tokens up.  Process-wide. */
int ghost_set_gram_pair_mode(int mode);

/* ---- train-gradient recovery ------------------------------------------------------------------- */
/* out[m_cols, n_cols] (= or +=) scale * sum_{row < n_rows} X[row, :]^T Y[row, :].
 * nn.Linear weight [d_out, d_in]: X = out-grad, Y = activations; HF Conv1D weight [d_in, d_out]:
 * X = activations, Y = out-grad.  ws: fp32 scratch of ghost_wgrad_workspace_bytes().
 * Replaces ghostEngines/supported_layers_grad_samplers_dotprod.py:155-173 and :474-506 together
 * with the batch-size rescale of ghostEngines/autograd_grad_sample_dotprod.py:132-134 (folded into
 * `scale`). */
long long ghost_wgrad_workspace_bytes(int m_cols, int n_cols);
int ghost_wgrad_bf16(const void* X, const void* Y, long long n_rows, int m_cols, int n_cols,
                     long long ldx, long long ldy, float scale, int accumulate, void* out,
                     int out_is_f32, void* ws, long long ws_bytes, void* stream);

/* ---- Linear / Conv1D weight dot product, per-sample-gradient path ---------------------------- */
/* X, Y: [n_train + n_val, T, cols] bf16.  M[v,b] = dot_scale * <X_v^T Y_v, X_b^T Y_b>.  Per-sample
 * weight-gradient tiles are formed in TMEM by a tcgen05 GEMM over each sample's tokens and written
 * tile-major to the workspace (bf16, or fp32 when v_is_f32); a streaming kernel then contracts the
 * validation tiles with the train tiles into M and, if grad_out != NULL, sums the train tiles into
 * the train gradient grad_scale * sum_b X_b^T Y_b in the same pass (so ghost_wgrad_bf16 is not
 * needed for that layer).  Train samples are processed in groups sized to the workspace.
 * Replaces ghostEngines/supported_layers_grad_samplers_dotprod.py:131-135 and :443-447, per
 * validation sample (the reference's version sums the validation batch first). */
long long ghost_persample_workspace_bytes(int n_train, int n_val, int m_cols, int n_cols, int v_is_f32);
/* Upper bound on that workspace (default 12 GiB); smaller values make the train samples go through
 * in more, smaller groups.  Process-wide; set it before sizing workspaces. */
int ghost_set_persample_budget_bytes(long long bytes);
/* Selects the kernel of the tile pass: 0 = one CTA per 128 x 256 tile; 1 (default) = a CTA pair
 * (tcgen05 cta_group::2) per 256 x 256 block when both operands have column counts that are
 * multiples of 64 and X's 128-column tile count is even or at least 15; 2 = the pair kernel
 * whenever the column counts allow it.  Both kernels store identical tiles.  Process-wide. */
int ghost_set_persample_pair_mode(int mode);
/* The same choice for ghost_wgrad_bf16's split-K pass (modes 0 / 1 / 2 as above; default 1). */
int ghost_set_wgrad_pair_mode(int mode);
/* colsum_of = 1 (X) or 2 (Y) also writes the per-sample column sums of that operand,
 * colsum_out[s, c] = sum_t operand[s, t, c] (fp32, [n_train + n_val, cols]): the bias terms of
 * ghostEngines/supported_layers_grad_samplers_dotprod.py:138-146, 454-471 without a second pass over
 * the out-grad: four extra warps of the GEMM kernel read the operand rows through L2 while the TMA
 * producer fetches the same rows for the tensor core (about 5 % on the GEMM call, less than the
 * separate ghost_colsum pass).  Only meaningful when the operand holds the values themselves (not the
 * hi/lo split of fp32 data); 0 = off. */
int ghost_persample_dot_bf16(const void* X, const void* Y, int n_train, int n_val, long long T,
                             int m_cols, int n_cols, long long ldx, long long ldy, float dot_scale,
                             float* M_out, int v_is_f32, void* grad_out, int grad_is_f32,
                             float grad_scale, int grad_accumulate, int colsum_of, float* colsum_out,
                             void* ws, long long ws_bytes, void* stream);

/* The same path as two calls, for callers that put something between the passes: in a data-parallel
 * run whose ranks each hold a part of the validation batch, a rank computes the tiles of its own
 * validation samples, all-gathers them (NCCL, into local memory), and then contracts all validation
 * tiles with its train tiles -- half the bytes of gathering the validation operands, and no rank
 * repeats another rank's validation GEMMs.
 *   ghost_persample_tiles_bf16: the tile pass for samples [sample0, sample0 + samples) of X, Y
 *     ([n_samples_total, T, cols] bf16) into tiles_out, laid out [tile][samples][128 x 256] bf16
 *     (ghost_persample_tiles_bytes, 256-byte aligned); colsum_of / colsum_out as above (rows sample0..).
 *   ghost_tile_dot_bf16: M_out[v, b] = dot_scale * <V_v, W_b> and, if grad_out != NULL, the train
 *     gradient grad_scale * sum_b W_b (bf16 only for n_train <= 32).  W: [tile][n_train][128 x 256];
 *     V: [v_ranks][tile][v_per_rank][128 x 256], what all_gather leaves (validation sample v of the
 *     result is sample v % v_per_rank of rank v / v_per_rank; v_ranks = 1 is a plain tile-major
 *     buffer).  v_per_rank must divide, or be a multiple of, the kernel's block of 8 / 16 / 32
 *     validation rows (8 up to 8 validation samples, 16 up to 16, else 32).
 * Same reference lines as ghost_persample_dot_bf16. */
long long ghost_persample_tiles_bytes(int samples, int m_cols, int n_cols);
int ghost_persample_tiles_bf16(const void* X, const void* Y, int n_samples_total, long long T, int m_cols,
                               int n_cols, long long ldx, long long ldy, int sample0, int samples,
                               int colsum_of, float* colsum_out, void* tiles_out, long long tiles_bytes,
                               void* stream);
int ghost_tile_dot_bf16(const void* V, int v_ranks, int v_per_rank, const void* W, int n_train, int m_cols,
                        int n_cols, float dot_scale, float* M_out, void* grad_out, int grad_is_f32,
                        float grad_scale, int grad_accumulate, void* stream);

/* ---- bias / LayerNorm / small reductions ------------------------------------------------------- */
/* out[n, c] = sum_t G[n, t, c]  (fp32).  Replaces the token sums of
 * ghostEngines/supported_layers_grad_samplers_dotprod.py:138-146, 454-471 and
 * ghostEngines/autograd_grad_sample_dotprod.py:199-222. */
int ghost_colsum(const void* G, int is_f32, int N, long long T, int cols, long long ld, float* out,
                 void* stream);
/* Per-sample LayerNorm parameter gradients in one pass over A and G:
 * gw[n,f] = sum_t G[n,t,f] * xhat[n,t,f], gb[n,f] = sum_t G[n,t,f], xhat = layer norm of A over the
 * last dim without affine.  Replaces
 * ghostEngines/supported_layers_grad_samplers_dotprod.py:262-300 and :347-363.
 * ws: scratch of ghost_layernorm_workspace_bytes() for the per-CTA partial sums, which are then
 * added in a fixed order (the result is run-to-run deterministic). */
long long ghost_layernorm_workspace_bytes(int N, long long T, int F);
int ghost_layernorm_persample(const void* A, const void* G, int is_f32, int N, long long T, int F,
                              float eps, float* gw, float* gb, void* ws, long long ws_bytes,
                              void* stream);
/* The same pass for an RMS norm (y = weight * x / sqrt(mean(x^2) + eps), no centring, no bias):
 * gw[n,f] = sum_t G[n,t,f] * x[n,t,f] / rms[n,t]; gsum[n,f] = sum_t G[n,t,f] is produced as well
 * (callers that do not need it pass scratch).  Workspace as for ghost_layernorm_persample.  The
 * reference has no RMS-norm support (ghostEngines/autograd_grad_sample_dotprod.py:76-79 skips such
 * layers with a warning), so Llama-style models get no dot products for their norm weights there. */
int ghost_rmsnorm_persample(const void* A, const void* G, int is_f32, int N, long long T, int F,
                            float eps, float* gw, float* gsum, void* ws, long long ws_bytes,
                            void* stream);
/* M[v,b] = scale * <X[n_train + v, :], X[b, :]> for per-sample vectors X[N, F] fp32.  Replaces the
 * einsum('p,bp->b') / einsum('bf,f->b') contractions of the bias and LayerNorm paths. */
int ghost_small_gram_f32(const float* X, int n_train, int n_val, int F, float scale, float* M_out,
                         void* stream);
/* out[c] (= or +=) scale * sum_{n < n_rows} X[n, c], cast to fp32 or bf16: averaged train gradient
 * of a bias / LayerNorm parameter from the per-sample vectors. */
int ghost_rows_sum(const float* X, int n_rows, int F, float scale, void* out, int out_is_f32,
                   int accumulate, void* stream);
/* Many of the two small reductions above in one launch.  Job j works on its layer's per-sample
 * vectors X[n_train + n_val, F] (fp32): M[v, b] = dot_scale * <X[n_train + v], X[b]> when M is not
 * NULL, and sum_out[c] = sum_scale * sum_{b < n_train} X[b, c] (fp32 or bf16) when sum_out is not
 * NULL.  `jobs` is a HOST array; its entries travel to the device as kernel parameters, 48 per
 * launch.  Replaces, for a whole backward pass at once, the per-layer einsum('bp,p->b') / sum(dim=0)
 * calls of ghostEngines/supported_layers_grad_samplers_dotprod.py:143-146, 281-300, 347-363 and
 * ghostEngines/autograd_grad_sample_dotprod.py:211-220. */
typedef struct ghost_small_job {
  const float* X;
  float* M;
  void* sum_out;
  int n_train, n_val, F;
  int sum_is_f32;
  float dot_scale, sum_scale;
  /* Validation rows kept apart from X (X then holds the train rows, and whatever follows them is
   * not read): validation row v is Xv[(v / v_per_rank) * v_rank_pitch + (v % v_per_rank) * F], the
   * layout of one all-gather over ranks that carried many jobs' validation rows at once (every
   * rank sent one packed buffer of v_rank_pitch floats; this job's rows start at Xv inside it).
   * Xv = NULL: the validation rows follow the train rows in X. */
  const float* Xv;
  long long v_rank_pitch;
  int v_per_rank;
} ghost_small_job;
int ghost_small_reduce_batch(const ghost_small_job* jobs, int n_jobs, void* stream);

/* ---- Embedding -------------------------------------------------------------------------------- */
/* M[v,b] = scale * sum_{t,s : ids_b[t] == ids_v[s]} <G_b[t], G_v[s]>.  ids: int64 [N, T]; G: [N, T, d].
 * Validation tokens are chained per id; a train token walks the chain of its id.  The workspace
 * must hold at least ghost_embedding_dot_workspace_bytes (the chain tables).  With
 * ghost_embedding_dot_workspace_bytes_for or more, ids that more than max(16, 4 * n_val) validation
 * tokens share (padding, separators; up to 256 such ids) are first summed per (id, validation
 * sample), so a train token costs at most n_val dot products however often its id repeats; with the
 * smaller workspace the work is sum over ids of count_train(id) * count_val(id) * d.  An id
 * outside [0, vocab) contributes nothing and makes the next ghost_poll_kernel_error return
 * GHOST_ERR_INDEX.  Replaces ghostEngines/supported_layers_grad_samplers_dotprod.py:181-211. */
long long ghost_embedding_dot_workspace_bytes(int n_val, long long T, int vocab);
long long ghost_embedding_dot_workspace_bytes_for(int n_val, long long T, int vocab, int d);
int ghost_embedding_dot(const long long* ids, const void* G, int is_f32, int n_train, int n_val,
                        long long T, int d, int vocab, float scale, float* M_out, void* ws,
                        long long ws_bytes, void* stream);
/* Same result as ghost_embedding_dot for callers that cannot supply a workspace because they are not
 * allowed to allocate device memory at that point (a process whose device memory belongs to a
 * fixed pool, or code running inside another component's critical section where re-entering any
 * allocator would deadlock).  The id-chain tables live in a 1 MiB __device__ array inside the
 * library (one copy per GPU that loads it, kept until exit), hence the limits vocab <= 131072 and
 * n_val * T <= 131072; anything larger returns GHOST_ERR_INVALID.  The call allocates nothing.  Its
 * first use on a device looks up the array's device address (cudaGetSymbolAddress) and should
 * come before any stream capture.  All calls on a GPU share the one array: calls that can overlap
 * on the device race, so keep them on one stream or order them.  No counterpart in the reference:
 * the reference allocates a [vocab, d] table on every call. */
int ghost_embedding_dot_noalloc(const long long* ids, const void* G, int is_f32, int n_train, int n_val,
                                long long T, int d, int vocab, float scale, float* M_out, void* stream);
/* out[vocab, d] (= or +=) round(sum over train tokens with that id of round(G * pre_scale)) / divisor
 * in the table dtype, accumulated in fp32 in ascending token order (bit-identical to the CPU
 * index_add_).  Replaces ghostEngines/supported_layers_grad_samplers_dotprod.py:214-235. */
long long ghost_embedding_wgrad_workspace_bytes(int n_train, long long T, int vocab);
int ghost_embedding_wgrad(const long long* ids, const void* G, int is_f32, int n_train, long long T,
                          int d, int vocab, float pre_scale, float divisor, int accumulate, void* out,
                          void* ws, long long ws_bytes, void* stream);

/* ---- GradProj ------------------------------------------------------------------------------------ */
/* out + b * out_stride <- scale * (G_b P_r^T)^T (A_b P_c^T), [k_r, k_c] fp32 row-major, for every
 * sample b.  G: [B, T, n_r], A: [B, T, n_c], P_r: [k_r, n_r], P_c: [k_c, n_c], all bf16.
 * nn.Linear: (G, P_r) = (out-grad, P_o), (A, P_c) = (activations, P_i).  HF Conv1D: the reference
 * projects the out-grad with P_i and the activations with P_o, i.e. P_r = P_i, P_c = P_o.
 * Replaces ghostEngines/gradProjection/autograd_gradproj.py:120-165 and the per-layer
 * reshape + cat of ghostEngines/gradProjection/gradproj_engine.py:240-263 (results land directly
 * in the caller's [B, total_proj_dim] slices). */
int ghost_gradproj_dense_bf16(const void* G, const void* A, int B, long long T, int n_r, int n_c,
                              long long ldg, long long lda, const void* P_r, const void* P_c, int k_r,
                              int k_c, long long ldpr, long long ldpc, float scale, float* out,
                              long long out_stride, void* stream);
/* out + b * out_stride + o * out_ld + i (+)= scale * sum_t (P_o g_bt)[o] * P_i[i, id_bt] for every sample
 * b, o < k_o, i < k_i: the projected gradient of an embedding table.  ids: [B, T] int64; G: [B, T, d]
 * out-grad rows (fp32 or bf16, row pitch ldg); P_o: bf16 [k_o, ldp_o] as ghost_cast_split_bf16 lays
 * it out -- bf16(P_o) in columns [0, p_cols), p_cols = d rounded up to a multiple of 8, and, for fp32
 * out-grads, the residual P_o - bf16(P_o) in columns [p_lo_offset, p_lo_offset + p_cols);
 * P_i_t: fp32 [vocab, >= k_i] with row pitch ld_pit, P_i transposed, so that a token id selects one
 * contiguous row.  k_o, k_i <= 64 per call: larger projections are covered block by block (row
 * offsets into P_o / out, column offsets into P_i_t / out, out_ld = the full k_i).  accumulate = 0
 * zeroes the samples' blocks first and needs out_ld == k_i.  An id outside [0, vocab) contributes
 * nothing and makes the next ghost_poll_kernel_error return GHOST_ERR_INDEX.
 * Replaces ghostEngines/gradProjection/autograd_gradproj.py:167-222 (a Python loop over all
 * tokens with one host synchronisation per token). */
int ghost_gradproj_embedding(const long long* ids, const void* G, int g_is_f32, int B, long long T, int d,
                             long long ldg, const void* P_o, long long ldp_o, int p_cols, int p_lo_offset,
                             const float* P_i_t, long long ld_pit, int vocab, int k_o, int k_i, float scale,
                             int accumulate, float* out, long long out_stride, int out_ld, void* stream);
/* S[n1, n2] (row pitch ld_s, fp32) <- scale * P1 P2^T for two blocks of projection rows
 * P1: [n1, D], P2: [n2, D] (both fp32 or both bf16, row pitches ld1, ld2).  Meant for batch-sized
 * blocks (tens of rows) against a very long D = total_proj_dim, where both operands are streamed
 * once; larger blocks are correct but re-read the operands once per 16 x 16 output block.
 * Replaces the proj1 @ proj2.t() of Examples/ghost_gradproj_lm.py:190-196 and
 * Examples/GradProj_LM/plot_error_with_dim.py:69-86 while the rows are still on the device. */
int ghost_projection_similarity(const void* P1, const void* P2, int is_f32, int n1, int n2, long long D,
                                long long ld1, long long ld2, float scale, float* S, long long ld_s,
                                void* stream);

/* ---- benchmark model helper (not part of the ghost hot path) ------------------------------------ */
/* Token cross-entropy of a [rows, cols] logit matrix whose last cols - cols_valid columns are padding
 * (they take no probability mass and get zero gradient).  Forward: lse[r] = log-sum-exp over the
 * valid columns, loss_rows[r] = lse[r] - logits[r, targets[r]] (0 where targets[r] == ignore_index);
 * one pass over the logits.  Backward: dlogits[r, c] = scale[0] * (softmax - onehot), scale a
 * device scalar (upstream gradient / number of counted rows); one read and one write.  Used by
 * the loss of the synthetic GPT-2 model the benchmark trains.  No counterpart in the reference,
 * whose models take their loss from torch ops. */
int ghost_workload_ce_forward(const void* logits, int is_f32, long long rows, int cols, int cols_valid,
                              long long ld, const long long* targets, long long ignore_index, float* lse,
                              float* loss_rows, const float* scale, void* dlogits, void* stream);
/* With dlogits != NULL the forward also writes scale[0] * (softmax - onehot) as dense [rows, cols]
 * (the gradient for an upstream gradient of 1 when scale = 1 / counted rows): its second pass over a
 * row hits L2.  ghost_workload_ce_rescale then multiplies by the actual upstream gradient in place
 * and returns at once when that is exactly 1. */
int ghost_workload_ce_rescale(void* dlogits, int is_f32, long long rows, int cols, const float* upstream,
                              void* stream);
int ghost_workload_ce_backward(const void* logits, int is_f32, long long rows, int cols, int cols_valid,
                               long long ld, const long long* targets, long long ignore_index,
                               const float* lse, const float* scale, void* dlogits, long long ld_out,
                               void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GHOST_B200_H_ */
