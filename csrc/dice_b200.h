// C interface of libdice_b200 (sm_100a): every exported entry point of the kernel library.
//
// All pointers are device pointers unless stated otherwise; `stream` is a cudaStream_t passed as void*.  A function
// returns 0 when its launch was accepted, a negative code when the arguments were rejected (-3 kernel attribute,
// -4 launch error, -5 alignment, -6 unsupported shape / model, -7..-9 see dice_positive_correction_noalloc).
// Device-side failures (bounded waits that gave up, indices out of range) are reported through the caller's status
// word: 0 ok, 1 producer / 2 MMA / 3 epilogue wait timed out, 4 peer wait timed out, 5 index out of range,
// 6 inbox overflow, 7 copy drain timed out.  Kernels that touch peer memory return at once when the status word
// already holds an error.  "table" arguments are device arrays of per-rank base pointers (peer memory allowed);
// "mc" arguments are addresses inside an NVSwitch multicast mapping (null selects the peer-pointer path).
// Entity row e of a row-sharded table lives on rank e % W at local row e / W.
// Model codes: 0 DistMult, 1 ComplEx, 2 QMult, 3 OMult, 4 Keci Cl(0,1), 5 translation (q = h + r).
// Optimiser kinds: 0 Adam, 1 AdamW, 2 SGD, 3 ADOPT.
#pragma once

#ifdef __CUDACC__
#include <cuda_bf16.h>
typedef __nv_bfloat16 dice_bf16;
#else
typedef unsigned short dice_bf16;   /* raw bits of a bfloat16 */
#endif

#ifdef __cplusplus
extern "C" {
#endif

// Optimiser step fused into dice_kvsall_fused: the launch that produces the last partial gradient of a 128-row tile of
// X applies Adam (kind 0), AdamW (1), SGD (2) or ADOPT (3) to that tile.  param / m / v: fp32 [x_rows, D]; shadow: the
// bf16 rows (the x operand itself); count: [ceil(x_rows / 128)] zero-initialised words (zero again afterwards);
// step: device counter of completed steps (read, not advanced).
typedef struct DiceFusedOptimizer {
  float* param;
  float* m;
  float* v;
  void* shadow;
  unsigned int* count;
  const long long* step;
  float lr, beta1, beta2, eps, weight_decay;
  int kind;
} DiceFusedOptimizer;

// ---------------------------------------------------------------------------------------- tensor-core scoring
// out[x_rows, D] += scale * (sigmoid(X Yᵀ) - label) * Y and, with_loss, *loss += sum softplus(s) - label * s; x, y bf16
// row-major, D in {64, 128, 256}.  Labels: `base` everywhere, base + pos_delta where the bit mask (row stride
// mask_stride words, a multiple of 4) is set.  trace (optional) receives int64[64][8] pipeline stamps of CTA 0.
// score_mode 0: logit = x.y; 1: x.y + x_bias[x] + y_bias[y]; 2: margin - sqrt(x_bias[x] + y_bias[y] - 2 x.y) (squared
// norms as biases; out then holds sum_y w y with w = dS / distance).  x_bias / y_bias: fp32, readable up to the next
// multiple of 128 rows, null = zeros; x_dsum (optional, [x_rows]) += scale * row sums of the second GEMM's A operand.
int dice_kvsall_fused(const void* x, int x_rows, const void* y, int y_rows, int D, float* out, double* loss,
                      float base, float scale, int with_loss, int* status, int num_ctas, const unsigned int* mask,
                      int mask_stride, float pos_delta, long long* trace, int score_mode, const float* x_bias,
                      const float* y_bias, float* x_dsum, float margin, const DiceFusedOptimizer* opt, void* stream);
// CTA-pair variant (tcgen05.mma.cta_group::2), D = 256.  loss_share -1 / 0 / 1: all / even / odd 256 x 256 blocks add
// their loss terms in this launch.  trace: optional int64[64][8] pipeline stamps.
int dice_kvsall_pair(const void* x, int x_rows, const void* y, int y_rows, int D, float* out, double* loss, float base,
                     float scale, int with_loss, int* status, int num_pairs, const unsigned int* mask,
                     int mask_stride, float pos_delta, int loss_share, long long* trace, void* stream);

// Filtered-rank counting / running top-k over X Yᵀ without storing it (see csrc/eval_rank.cu).
int dice_eval_rank(const void* x, int x_rows, const void* y, int y_rows, int D, const float* target,
                   const int* target_idx, const float* col_bias, int y_offset, int y_stride, int* greater, int k,
                   int cand_cap, float* cand_score, int* cand_idx, int* cand_count, int* status, int num_ctas,
                   const float* margin, int* band_rows, int* band_cols, unsigned long long* band_count,
                   long long band_cap, float* row_floor, void* stream);
int dice_eval_rank_cand_cap(int x_rows, int y_rows, int D, int k, int num_ctas);
int dice_eval_sparse(const void* q, const void* y, int n, int D, int y_rows, int y_offset, int y_stride,
                     const int* target, const float* col_bias, const float* target_in, const long long* filt_ptr,
                     const int* filt_cols, float* target_score, int* filtered_greater, int fp32_operands, void* stream);
int dice_eval_band_exact(const float* q, const float* y, int D, int y_rows, int y_offset, int y_stride,
                         const float* col_bias, const int* band_rows, const int* band_cols,
                         const unsigned long long* band_count, long long band_cap, const float* target, int* greater,
                         void* stream);
// Cross-rank merges of the sharded evaluation by peer loads.
int dice_peer_sum_f32(const float* const* table, int W, float* out, int n, const int* status, void* stream);
int dice_merge_ranks(const int* const* greater, const int* const* filtered, int W, long long* ranks, int n,
                     const int* status, void* stream);
int dice_merge_topk(const float* const* score, const long long* const* idx, int W, int k, long long stride,
                    float* out_s, long long* out_i, int n, const int* status, void* stream);

// ---------------------------------------------------------------------------------------- lookup / composition
int dice_lookup_vec_supported(int model, int D);
int dice_lookup_compose_vec(int model, int normalize, const long long* idx_h, const long long* idx_r, int idx_stride,
                            const long long* dp_src, const float* const* ent, int W, long long num_entities,
                            int num_relations, const float* rel, const float* coeff, dice_bf16* const* q_dst,
                            int n_dst, void* q_mc, long long q_row_offset, float* q_f32, long long* const* ids_dst,
                            long long ids_stride, int B, int D, int* status, void* stream);
int dice_compose_backward_owner(int model, int normalize, const long long* idx_h, const long long* idx_r,
                                int idx_stride, const float* ent_local, int W, int rank, long long num_entities,
                                int num_relations, const float* rel, const float* coeff, const float* dq,
                                const float* const* dq_table, int n_dq, const void* dq_mc, float* g_ent_local,
                                float* g_rel, float* g_coeff, int n, int D, int* status, void* stream);
// Reduce-scatter of the partial query gradients alone.  dice_owned_rows compacts the batch rows whose head this rank
// owns into list[0 .. *count) (count zeroed by the caller); dice_dq_pull_owner then sets dq_local[i] = sum over the n_dq
// buffers of dq_table (peer loads) for the listed rows, in place.  Light enough to run beside a scoring launch.
int dice_owned_rows(const long long* idx_h, int idx_stride, int n, int W, int rank, long long num_entities, int* list,
                    int* count, int* status, void* stream);
int dice_dq_pull_owner(const int* list, const int* count, const float* const* dq_table, int n_dq, float* dq_local, int D,
                       int* status, void* stream);
// Scalar-per-thread variants (any D; used by the sampled engines and the collective-library comparison pipeline).
int dice_lookup_compose(int model, int normalize, const long long* idx_h, const long long* idx_r,
                        const float* const* ent, int W, long long num_entities, const float* rel, const float* coeff,
                        dice_bf16* const* q_dst, int n_dst, long long q_row_offset, float* q_f32, int B, int D, int* status,
                        const long long* dp_src, long long* const* dp_dst, void* stream);
int dice_compose_backward(int model, int normalize, const long long* idx_h, const long long* idx_r,
                          const float* const* ent, int W, const float* rel, const float* coeff, const float* dq,
                          float* const* g_ent, float* g_rel, float* g_coeff, int B, int D,
                          unsigned char* const* touched, const float* const* dq_table, int n_dq,
                          long long dq_row_offset, void* stream);

// ---------------------------------------------------------------------------------------- labels
int dice_build_label_masks(const long long* dp_idx, const long long* offsets, const long long* values, int n, int W,
                           int rank, unsigned int* mask_q, int stride_q, unsigned int* mask_e, int stride_e,
                           void* stream);
// first == null: one launch with block-local prefix sums; else count / scan / spread with first = int[n + 1] scratch.
int dice_build_label_masks_flat(const long long* dp_idx, const long long* offsets, const long long* values, int* first,
                                int n, int W, int rank, unsigned int* mask_q, int stride_q, unsigned int* mask_e,
                                int stride_e, long long num_data_points, long long num_local_rows, int* status,
                                void* stream);

// Largest batch (number of data points) the allocation-free entry point accepts.
#define DICE_NOALLOC_MAX_BATCH 65536

int dice_positive_scan(const long long* dp_idx, const long long* offsets, int n, int* first, void* stream);

int dice_positive_correction(const long long* dp_idx, const long long* offsets, const long long* values,
                             const int* first, const void* q, const void* e, float* dq, float* de, double* loss,
                             float weight, float scale, int n, int D, int W, int rank, float* const* dq_table,
                             int dq_block_rows, void* stream);

// Allocation-free variant of dice_positive_scan + dice_positive_correction.  This entry point has no counterpart in
// the reference implementation (which has no native code at all); it exists for callers that cannot allocate
// device memory: the int[n + 1] prefix-sum scratch lives in a fixed __device__ array inside the library
// (DICE_NOALLOC_MAX_BATCH + 1 ints per GPU that loads the library).  n > DICE_NOALLOC_MAX_BATCH returns -7.
// The first call on a device resolves the array's device address and should happen before any stream capture.
// Calls share the array: calls that overlap on the GPU race and must be serialised by the caller.
int dice_positive_correction_noalloc(const long long* dp_idx, const long long* offsets, const long long* values,
                                     const void* q, const void* e, float* dq, float* de, double* loss, float weight,
                                     float scale, int n, int D, int W, int rank, void* stream);

// ---------------------------------------------------------------------------------------- sampled scoring
int dice_uniform_int(long long* out, long long n, long long high, unsigned long long seed, unsigned long long offset,
                     const long long* step_ptr, long long out_stride, long long row_len, void* stream);
int dice_neg_sample(const long long* pos, int B, int k, long long num_entities, unsigned long long seed,
                    unsigned long long offset, const long long* step_ptr, int mode, float label_pos, float label_neg,
                    long long* x, long long* h, long long* r, long long* t, float* y, void* stream);
int dice_candidate_bce(const float* q, const long long* cand, long long cand_stride, long long cand_step, int C,
                       const float* labels, const float* const* ent, float* const* g_ent, float* dq, float* scores,
                       double* loss, float scale, int kind, float margin, float eps, int N, int D, int W,
                       unsigned char* const* touched, long long num_entities, int* status, void* stream);

// ---------------------------------------------------------------------------------------- optimisers, step bookkeeping
int dice_optimizer_step(int kind, float* param, float* grad, float* m, float* v, void* shadow, const long long* step,
                        long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                        const float* const* grad_table, int n_grad, const float* grad_mc, const int* status,
                        void* stream);
int dice_sparse_rows_optimizer(int kind, float* param, float* grad, float* m, float* v, void* shadow,
                               unsigned char* touched, long long rows, int D, const long long* step, float lr,
                               float beta1, float beta2, float eps, float weight_decay, void* stream);
// Host arrays of n_seg <= 3 segment descriptors; the last block closes the step when `done` is given.
int dice_step_tail(int kind, int n_seg, float* const* param, float* const* grad, float* const* m, float* const* v,
                   void* const* shadow, const long long* n, const float* const* const* grad_table,
                   const float* const* grad_mc, int n_grad, long long* step, float lr, float beta1, float beta2,
                   float eps, float weight_decay, double* acc, float* loss_out, double inv_count,
                   const double* const* acc_table, int n_acc, unsigned int* done, const int* status, void* stream);
// Two-shot all-reduce of a gradient slice + optimiser update + broadcast of the updated parameters.
int dice_bucket_reduce_update(int kind, float* const* p_dst, void* p_mc, const float* p_local,
                              const float* const* g_src, const void* g_mc, float* m, float* v, const long long* step,
                              long long lo, long long hi, int W, float lr, float beta1, float beta2, float eps,
                              float weight_decay, float grad_scale, const int* status, void* stream);
int dice_finish_step(double* acc, float* loss_out, double inv_count, long long* step, const double* const* acc_table,
                     int n_acc, const int* status, void* stream);
int dice_cast_bf16(const float* src, void* dst, long long n, void* stream);
int dice_timestamp(unsigned long long* slot, void* stream);
// Bounded barrier over W ranks on per-rank signal arrays in peer memory (spin_limit 0 = default).
int dice_p2p_barrier(unsigned int* const* sig_table, int rank, int W, unsigned int* count, int* status,
                     unsigned int spin_limit, void* stream);

// ---------------------------------------------------------------------------------------- convolutional gate
// 3x3 convolution with one input channel, batch normalisation and ReLU of the ConEx / ConvQ / ConvO families.
int dice_conv_gate_supported(int B, int H, int W, int C);
int dice_conv_gate_forward(int B, int H, int W, int C, int training, const float* X, const float* w,
                           const float* bias, const float* gamma, const float* beta, float* run_mean, float* run_var,
                           float momentum, float eps, double* stats, float* fold, float* F, void* stream);
int dice_conv_gate_backward(int B, int H, int W, int C, int training, const float* X, const float* w,
                            const float* bias, const float* fold, const float* dF, double* bstats, float* dX,
                            double* dwb, void* stream);

#ifdef __cplusplus
}
#endif
