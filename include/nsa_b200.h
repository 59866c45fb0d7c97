/* C ABI of libnsa_b200.so: the NSA (native sparse attention) hot path on B200.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*; 0 = the legacy default stream), launches asynchronously on
 * that stream and returns 0 on success or a negative NSA_ERR_* code.  After a
 * failure nsa_last_error() returns a description (thread-local).  No entry
 * point allocates device memory unless its comment says so: scratch space is
 * passed in by the caller and sized by the matching *_workspace_bytes call.
 *
 * Tensor layouts (all contiguous, row-major):
 *   q, o, do, dq          [B, Hq,  T,  D]
 *   k, v, dk, dv          [B, Hkv, Lk, D]   Lk = T (window, selection) or n_blk (compression)
 *   lse                   [B, Hq,  T]       float32, natural log; -1e9 on rows that attend nothing
 *   block_idx             [B, Hkv, T,  S]   int32, -1 = empty slot
 *   gate_logits           [B, Hq,  T,  3]
 * Query head h reads kv head h / (Hq / Hkv).  Scores are scaled by D^-1/2.
 *
 * "Reference" below is the msb-msb/openbox-llm checkout; citations are
 * file:line inside it.
 */
#ifndef NSA_B200_H
#define NSA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NSA_DTYPE_BF16 0
#define NSA_DTYPE_F32  1

#define NSA_MODE_WINDOW   0   /* nsa_fused_kernel.py:46 */
#define NSA_MODE_COMPRESS 1   /* nsa_fused_kernel.py:47 */
#define NSA_MODE_COMPRESS_STRIDED 3   /* no counterpart in the reference: `window` is the summary stride */

/* which kernel family serves a call */
#define NSA_IMPL_AUTO 0   /* tcgen05 kernels when the shape allows, else the SIMT kernels */
#define NSA_IMPL_SIMT 1   /* CUDA-core kernels: any dtype, D in {16,32,64,128}, any G and block size */
#define NSA_IMPL_TC   2   /* tcgen05/TMEM kernels only; NSA_ERR_UNSUPPORTED if the shape does not fit */

#define NSA_OK               0
#define NSA_ERR_BAD_ARG     -1
#define NSA_ERR_UNSUPPORTED -2
#define NSA_ERR_CUDA        -3
#define NSA_ERR_WORKSPACE   -4
#define NSA_ERR_DEVICE_WAIT -5   /* a bounded wait inside a kernel ran out */

typedef struct NsaDims {
  int32_t B, Hq, Hkv, T, D;
  int32_t dtype;            /* NSA_DTYPE_* of q,k,v,o and their gradients */
} NsaDims;

const char* nsa_last_error(void);
int nsa_version(void);
/* 1 if the tcgen05 kernels can serve this shape (bf16, D in {64,128}, Hq/Hkv in {1,2,4,8,16}...) */
int nsa_tc_supported(const NsaDims* dims, int block_size);

/* ---- range attention: sliding window and compressed-KV branches --------------------------
 * Replaces _range_attn_forward / _range_attn_backward and the kernels under them
 * (nsa_fused_kernel.py:442-518, kernels :61-426) behind _RangeAttn (:521-534).
 * mode WINDOW: query t attends keys [max(0,t-window+1), t]; Lk = T.
 * mode COMPRESS: query t attends summaries j with (j+1)*block_size-1 <= t; Lk = n_blk (`window`
 *   is ignored, as in the reference).
 * mode COMPRESS_STRIDED: `window` is a summary stride d <= block_size: summary j covers tokens
 *   [j*d, j*d + block_size) and is attended when j*d + block_size - 1 <= t; d = block_size is
 *   mode COMPRESS.
 * The forward also writes lse (the reference recomputes it in backward). */
/* Backward of a gated branch: when row_scale / row_dot [B,Hq,T] float32 are given (both or
 * neither), d_o is the upstream gradient of the whole op, the branch's own gradient is
 * row_scale * d_o and its delta is row_scale * row_dot, row_dot = sum_d d_o * o_branch; o is then
 * not read.  nsa_gate_combine_bwd_rows produces both arrays for the three branches. */
int nsa_range_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                       const NsaDims* dims, int Lk, int mode, int window, int block_size,
                       int impl, void* stream);
size_t nsa_range_attn_bwd_workspace_bytes(const NsaDims* dims, int Lk, int mode, int window, int impl);
int nsa_range_attn_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                       const void* d_o, void* dq, void* dk, void* dv,
                       const NsaDims* dims, int Lk, int mode, int window, int block_size,
                       const float* row_scale, const float* row_dot,
                       void* workspace, size_t workspace_bytes, int impl, void* stream);

/* ---- selected-block attention --------------------------------------------------------------
 * Replaces selection_forward_triton (nsa_selection_kernel.py:175-213, kernels :104-291 and
 * the LSE combine :336-365) and selection_backward_triton / selection_backward_fsa
 * (nsa_selection_backward.py:156-189, :278-334) behind SelectionAttnTriton (:337-365).
 * Query i attends token pos = blk*block_size+n of every listed block with blk >= 0,
 * pos <= i and pos < T (nsa_selection_kernel.py:144). */
size_t nsa_selection_fwd_workspace_bytes(const NsaDims* dims, int S, int block_size, int impl);
int nsa_selection_fwd(const void* q, const void* k, const void* v, const int32_t* block_idx,
                      void* o, float* lse, const NsaDims* dims, int S, int block_size,
                      void* workspace, size_t workspace_bytes, int impl, void* stream);
size_t nsa_selection_bwd_workspace_bytes(const NsaDims* dims, int S, int block_size, int impl);
int nsa_selection_bwd(const void* q, const void* k, const void* v, const int32_t* block_idx,
                      const void* o, const float* lse, const void* d_o,
                      void* dq, void* dk, void* dv, const NsaDims* dims, int S, int block_size,
                      const float* row_scale, const float* row_dot,
                      void* workspace, size_t workspace_bytes, int impl, void* stream);

/* The tcgen05 selection kernels walk the block list block by block: CSR (nsa_fsa.py:14-64), the
 * (query, slot) -> pair map and a work list, which nsa_selection_fwd and nsa_selection_bwd each
 * build inside their workspace.  A caller that runs both on one block list (every training step)
 * can build them once into a buffer of nsa_selection_plan_bytes bytes (0: shape not served by the
 * tcgen05 kernels) and hand it to the *_planned forms, which copy it into place instead of
 * building.  The reference builds its CSR once per forward and once per backward
 * (nsa_selection_kernel.py:199-201, nsa_selection_backward.py:356-358); no counterpart for the
 * reuse. */
size_t nsa_selection_plan_bytes(const NsaDims* dims, int S, int block_size);
int nsa_selection_plan_build(const int32_t* block_idx, const NsaDims* dims, int S, int block_size,
                             void* plan, size_t plan_bytes, void* stream);
int nsa_selection_fwd_planned(const void* q, const void* k, const void* v, const int32_t* block_idx,
                              void* o, float* lse, const NsaDims* dims, int S, int block_size,
                              void* workspace, size_t workspace_bytes, const void* plan, void* stream);
int nsa_selection_bwd_planned(const void* q, const void* k, const void* v, const int32_t* block_idx,
                              const void* o, const float* lse, const void* d_o,
                              void* dq, void* dk, void* dv, const NsaDims* dims, int S, int block_size,
                              const float* row_scale, const float* row_dot,
                              void* workspace, size_t workspace_bytes, const void* plan, void* stream);

/* dq of the whole op in one pass (no counterpart in the reference, which adds the three branch
 * gradients with torch).  When the tcgen05 kernels serve a backward call (nsa_tc_supported) its
 * `dq` argument may be NULL: the branch's bf16 dQ partials then stay in the call's workspace, and
 * this entry point adds the partials of the compression, selection and window branches of every
 * query in fp32 and writes dq [B,Hq,T,D] once.  ws_* are the workspaces of the three backward
 * calls (same dims; Lk_cmp, the summary length and stride, S, the selection block size and the
 * window as given to them); NULL = branch absent. */
int nsa_dq_reduce3(const NsaDims* dims, int Lk_cmp, int cmp_len, int cmp_stride, int S, int block_size,
                   int window, const void* ws_cmp, const void* ws_slc, const void* ws_win, void* dq,
                   void* stream);

/* The same without partial buffers for the window and compression branches (tcgen05 shapes only;
 * no counterpart in the reference, whose q-tiled backward kernels store dQ per query tile,
 * nsa_fused_kernel.py:420-425).  nsa_range_attn_bwd_acc is nsa_range_attn_bwd with the branch's
 * dQ ADDED, tile by tile (TMA reduce-add), to dq_acc, an fp32 buffer [B*Hkv][T][Hq/Hkv][D] that
 * the caller has zeroed and may hand to both branches in turn; its workspace
 * (nsa_range_attn_bwd_acc_workspace_bytes) then holds no partials.  nsa_dq_finish adds the
 * selection branch's partials (ws_slc: the workspace of an nsa_selection_bwd call with dq = NULL,
 * or NULL) to the accumulator and writes dq [B,Hq,T,D] in the input dtype.  The adds into dq_acc
 * happen in no fixed order, so dq can differ in its last bits from run to run; nsa_dq_reduce3 is
 * the bit-reproducible form. */
size_t nsa_range_attn_bwd_acc_workspace_bytes(const NsaDims* dims, int Lk, int mode, int window);
int nsa_range_attn_bwd_acc(const void* q, const void* k, const void* v, const void* o, const float* lse,
                           const void* d_o, float* dq_acc, void* dk, void* dv, const NsaDims* dims,
                           int Lk, int mode, int window, int block_size,
                           const float* row_scale, const float* row_dot,
                           void* workspace, size_t workspace_bytes, void* stream);
int nsa_dq_finish(const NsaDims* dims, int S, int block_size, const float* dq_acc, const void* ws_slc,
                  void* dq, void* stream);

/* ---- block -> query CSR ---------------------------------------------------------------------
 * Replaces build_block_to_query_csr (nsa_fsa.py:14-64): pairs (query i, block j) with j >= 0
 * and j*block_size <= i, grouped by (b, hkv, j), queries ascending.  block_offsets is
 * [B,Hkv,n_blk+1] global offsets; q_of_block and pair_bh need room for B*Hkv*T*S entries.
 * The number of pairs is block_offsets[B*Hkv*(n_blk+1)-1]. */
size_t nsa_csr_workspace_bytes(int B, int Hkv, int T, int S, int block_size);
int nsa_build_block_to_query_csr(const int32_t* block_idx, int B, int Hkv, int T, int S,
                                 int block_size, int32_t* q_of_block, int32_t* block_offsets,
                                 int32_t* pair_bh, void* workspace, size_t workspace_bytes,
                                 void* stream);

/* The same CSR for callers that may not allocate device memory and have no scratch buffer to
 * hand over: code running under a memory arena it does not own (an inference server's fixed
 * pool, a plugin loaded into another framework's process), or a latency-critical thread that
 * must not reach the driver's allocator, where a cudaMalloc can block on other streams' work.
 * The scratch is a fixed array inside the library, nsa_csr_builtin_scratch_bytes() (8 MiB) per
 * GPU that loads the library, held until the process exits; shapes whose
 * nsa_csr_workspace_bytes exceeds it are refused with NSA_ERR_WORKSPACE and a message.  The
 * call allocates nothing (no cudaMalloc / cudaFree, no allocating library routine); inputs and
 * the three outputs are still the caller's.  The first call on a device looks up the array's
 * device address (with lazy module loading that lookup is also what makes the driver bring the
 * module and its 8 MiB array onto the device, so "allocates nothing" holds from the second call
 * on); make that call outside any stream capture.  The device that is current at the call is the
 * one whose array is used: `stream` must belong to it.  The address cache is safe against
 * concurrent first calls from several host threads; it does not survive cudaDeviceReset.  All
 * calls on a device share the one array: it is cleared at the start of every call, and two calls whose kernels may overlap
 * on the GPU (different streams, no ordering between them) would corrupt each other.
 * This entry point has no counterpart in the reference. */
size_t nsa_csr_builtin_scratch_bytes(void);
int nsa_build_block_to_query_csr_noalloc(const int32_t* block_idx, int B, int Hkv, int T, int S,
                                         int block_size, int32_t* q_of_block,
                                         int32_t* block_offsets, int32_t* pair_bh, void* stream);

/* ---- compression summaries ------------------------------------------------------------------
 * Mean pooling replaces block_mean_pool (nsa_fused_kernel.py:549-554); the learned pooling
 * replaces BlockCompressor.forward (nsa_model.py:118-123) as called at nsa_model.py:336-337:
 * out = proj_w @ sum_pos softmax(pool_logits)[pos] * (x[pos] + intra_pos[pos]).
 * x [B,Hkv,T,D] -> out [B,Hkv,n_blk,D], n_blk = T / block_size.  Parameters are float32. */
int nsa_block_mean_pool_fwd(const void* x, void* out, int B, int Hkv, int T, int D, int block_size,
                            int dtype, void* stream);
int nsa_block_mean_pool_bwd(const void* d_out, void* dx, int B, int Hkv, int T, int D,
                            int block_size, int dtype, void* stream);
int nsa_block_compress_fwd(const void* x, const float* intra_pos, const float* pool_logits,
                           const float* proj_w, void* out, int B, int Hkv, int T, int D,
                           int block_size, int dtype, void* stream);
size_t nsa_block_compress_bwd_workspace_bytes(int B, int Hkv, int T, int D, int block_size);
int nsa_block_compress_bwd(const void* x, const float* intra_pos, const float* pool_logits,
                           const float* proj_w, const void* d_out, void* dx, float* d_intra_pos,
                           float* d_pool_logits, float* d_proj_w, int B, int Hkv, int T, int D,
                           int block_size, int dtype, void* workspace, size_t workspace_bytes,
                           void* stream);

/* The same learned pooling over windows of block_size tokens every `stride` tokens
 * (stride <= block_size; (T - block_size) / stride + 1 summaries): the compression geometry of the
 * published NSA recipe (length 32, stride 16).  No counterpart in the reference, whose
 * BlockCompressor is applied to a non-overlapping block view (nsa_model.py:217-220);
 * stride == block_size is exactly nsa_block_compress_fwd / _bwd. */
int nsa_block_compress_strided_fwd(const void* x, const float* intra_pos, const float* pool_logits,
                                   const float* proj_w, void* out, int B, int Hkv, int T, int D,
                                   int block_size, int stride, int dtype, void* stream);
size_t nsa_block_compress_strided_bwd_workspace_bytes(int B, int Hkv, int T, int D, int block_size,
                                                      int stride);
int nsa_block_compress_strided_bwd(const void* x, const float* intra_pos, const float* pool_logits,
                                   const float* proj_w, const void* d_out, void* dx,
                                   float* d_intra_pos, float* d_pool_logits, float* d_proj_w, int B,
                                   int Hkv, int T, int D, int block_size, int stride, int dtype,
                                   void* workspace, size_t workspace_bytes, void* stream);

/* ---- block scoring and top-n ----------------------------------------------------------------
 * Replaces the dense scoring pass of nsa_model.py:343-355: importance of block j for
 * (b, hkv, t) is the sum over the group's query heads of the compression-branch softmax
 * probability of summary j; the n_sel causally valid blocks ((j+1)*block_size-1 <= t) of
 * largest importance are written in order (importance descending, index ascending on ties),
 * -1 in slots with no valid block.  lse_cmp is the lse written by nsa_range_attn_fwd in
 * COMPRESS mode.  importance_out (optional, may be NULL) receives [B,Hkv,T,n_blk] float32. */
int nsa_topn_blocks(const void* q, const void* k_cmp, const float* lse_cmp, int32_t* block_idx,
                    float* importance_out, const NsaDims* dims, int n_blk, int block_size,
                    int n_sel, int impl, void* stream);

/* The same with forced blocks, as in the published NSA recipe ("always the initial block and the
 * local blocks"); no counterpart in the reference, whose scorer has none (nsa_model.py:257-258
 * takes a plain topk).  For query t, cur = t / block_size: the blocks j < n_init (with j <= cur)
 * come first in ascending order, then the n_local most recent blocks cur, cur-1, ... (the block
 * holding t is attended causally by the selection kernels), then the remaining slots by
 * importance as above.  n_init = n_local = 0 is nsa_topn_blocks. */
int nsa_topn_blocks_forced(const void* q, const void* k_cmp, const float* lse_cmp, int32_t* block_idx,
                           float* importance_out, const NsaDims* dims, int n_blk, int block_size,
                           int n_sel, int n_init, int n_local, int impl, void* stream);

/* The same when the compression summaries and the selection blocks sit on different grids (the
 * published NSA recipe: summaries of 32 tokens every 16, selection blocks of 64); no counterpart in
 * the reference, where the three sizes are one number.  k_cmp holds n_cmp summaries of cmp_len
 * tokens every cmp_stride tokens (lse_cmp from mode COMPRESS_STRIDED); cmp_len and sel_block are
 * multiples of cmp_stride.  The importance of selection block b is the sum of the importances of
 * the summaries that overlap it, and b is a candidate for query t once the first of them is
 * visible; forced blocks as above with cur = t / sel_block.  importance_out (optional) receives
 * the block importance [B,Hkv,T,ceil(T/sel_block)] (with the three sizes equal: [B,Hkv,T,n_cmp],
 * which is nsa_topn_blocks_forced). */
int nsa_topn_blocks_general(const void* q, const void* k_cmp, const float* lse_cmp, int32_t* block_idx,
                            float* importance_out, const NsaDims* dims, int n_cmp, int cmp_len,
                            int cmp_stride, int sel_block, int n_sel, int n_init, int n_local, int impl,
                            void* stream);

/* ---- projection glue ---------------------------------------------------------------------------
 * The reference layer runs seven projections and a gate projection as eight GEMMs and brings each
 * result to head-major layout by its own transpose + copy (nsa_model.py:192-194, 325-329, 358-359,
 * 366-367), and the output back by another (:369).  Here the eight weights are applied as ONE GEMM
 * whose rows [B,T,W] hold, per token, q (Hq*D), kc, vc, ks, vs, kw, vw (Hkv*D each) and the gate
 * logits (3*Hq, padded to a multiple of 8 elements: W = nsa_fused_projection_width);
 * nsa_split_heads turns those rows into q [B,Hq,T,D], kv [6,B,Hkv,T,D] and gate [B,Hq,T,3] in one
 * pass, nsa_merge_heads assembles the gradient rows from dq, dkv, dgate in one pass, and
 * nsa_swap_heads_tokens converts [B,H,T,D] <-> [B,T,H,D] (the op's output for out_proj, its upstream
 * gradient back). */
int nsa_fused_projection_width(int Hq, int Hkv, int D);
int nsa_split_heads(const void* y, void* q, void* kv, void* gate, int B, int T, int Hq, int Hkv, int D,
                    int dtype, void* stream);
int nsa_merge_heads(const void* dq, const void* dkv, const void* dgate, void* dy, int B, int T, int Hq,
                    int Hkv, int D, int dtype, void* stream);
int nsa_swap_heads_tokens(const void* src, void* dst, int B, int H, int T, int D, int dtype, int to_tokens,
                          void* stream);

/* ---- gate combine ---------------------------------------------------------------------------
 * Replaces the sigmoid blend nsa_model.py:366-368 / nsa_fused_kernel.py:572-573 and its
 * autograd backward: out = sum_i sigmoid(gate[...,i]) * o_i; d_gate is float32-accumulated
 * and written in the gate dtype. */
int nsa_gate_combine_fwd(const void* o_cmp, const void* o_slc, const void* o_win,
                         const void* gate_logits, void* out, const NsaDims* dims, void* stream);
int nsa_gate_combine_bwd(const void* o_cmp, const void* o_slc, const void* o_win,
                         const void* gate_logits, const void* d_out, void* do_cmp, void* do_slc,
                         void* do_win, void* d_gate_logits, const NsaDims* dims, void* stream);

/* Row statistics of the gate backward for the fused op: row_scale[3][B*Hq*T] = sigmoid(gate) and
 * row_dot[3][B*Hq*T] = <d_out, o_branch> (branch order cmp, slc, win), and d_gate_logits. */
int nsa_gate_combine_bwd_rows(const void* o_cmp, const void* o_slc, const void* o_win,
                              const void* gate_logits, const void* d_out, float* row_scale,
                              float* row_dot, void* d_gate_logits, const NsaDims* dims, void* stream);

/* out = a + b + c over n elements (fp32 accumulation): the sum of the three branches' dq that
 * autograd forms when one q feeds three branch Functions (nsa_model.py:330,338,360). */
int nsa_sum3(const void* a, const void* b, const void* c, void* out, size_t n, int dtype, void* stream);

/* ---- optimizer step of the data-parallel training step ---------------------------------------
 * Replace torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW of the reference's step
 * (train.py:148-149, :262-264) on flat fp32 buffers, with no host synchronisation in between.
 * nsa_sumsq_f32 adds sum(x^2) to *accum (device, zeroed by the caller).  nsa_adamw_step_f32 scales
 * the gradient by grad_scale (1 / world size after a summing all-reduce) and by the clip factor
 * min(1, max_norm / (grad_scale * sqrt(*sumsq) + 1e-6)) (sumsq NULL or max_norm <= 0: no clip), then
 * applies AdamW with decoupled weight decay and bias correction for `step` (counted from 1). */
int nsa_sumsq_f32(const float* x, size_t n, float* accum, void* stream);
int nsa_adamw_step_f32(float* p, const float* g, float* m, float* v, size_t n, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step, const float* sumsq,
                       float max_norm, float grad_scale, void* stream);

/* ---- accounting ------------------------------------------------------------------------------
 * nsa_launch_count: kernels launched by this library in this process so far.
 * nsa_profile_enable(1) makes every later kernel launch be bracketed by CUDA events on its own
 * stream (and drops earlier records); nsa_profile_summary waits for those events and writes one
 * line "kernel_name launches total_ms" per kernel into buf, returning the number of lines.
 * No counterpart in the reference (it times whole calls with perf_counter, bench_kernel.py:56-69). */
long long nsa_launch_count(void);
void nsa_profile_enable(int on);
int nsa_profile_summary(char* buf, size_t cap);

/* Tuning switches.  "sel_fwd_variant": 0 = the selection forward picks, on the device, between
 * its query-outer kernel (cheap when neighbouring queries share blocks) and its block-outer
 * kernel (cheap when they do not); 1 / 2 force one of them.  No counterpart in the reference
 * beyond its USE_FSA_FWD module flag (nsa_selection_kernel.py:48).
 * "debug_starve_load" (0 / 1, tests only): with 1 the tcgen05 window / compression / query-outer
 * forward kernel never sends the load of its second V tile, so that CTA's bounded wait runs out
 * after about a second: it raises the status word, waits for what it has in flight, gives its
 * tensor memory back and returns without writing.  This is how the give-up path is exercised
 * without faulting or hanging anything. */
int nsa_set_option(const char* name, int value);

/* Error word of the current device, raised by a kernel whose bounded wait ran out (0 = none).
 * Reading it synchronises the stream, returns NSA_ERR_DEVICE_WAIT when it was set and clears it.
 * While the word is set every tcgen05 kernel returns at entry and leaves its outputs unwritten, so
 * a caller that launches many steps without looking should read it at its own synchronisation
 * points.  The kernels of the reference have no status return (Python asserts only). */
int nsa_device_status(void* stream);

/* Sets the error word from the host (stream-ordered).  For tests of the give-up path: with the
 * word set, a launch returns without touching its outputs and nsa_device_status reports it, all
 * without making any kernel wait.  No counterpart in the reference. */
int nsa_debug_set_device_status(int value, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NSA_B200_H */
