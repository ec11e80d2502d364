// C ABI of the conef_b200 native library (sm_100a).
//
// Every entry point takes raw device pointers plus the CUDA stream to launch
// on, returns 0 on success and a non-zero code on failure (the message is
// available through conef_last_error()).  Nothing here allocates device
// memory except the functions whose name says so (conef_ipc_*); callers own
// all buffers.  The Python package binds these with ctypes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// One compressed (n x m) matrix living inside a flat gradient bucket.
// Offsets are in elements.  The sketch of the matrix is an (n x W) block in a
// flat sketch arena; its column hash table (m packed int32 entries:
// bucket | sign<<31) and its per-bucket column counts (W entries) live in flat
// int32 arenas.
typedef struct ConefMat {
  long long g_off;    // matrix start inside the bucket
  long long p_off;    // (n x r) block inside the flat P memory
  long long q_off;    // (m x r) block inside the flat Q memory
  long long sk_off;   // (n x W) block inside the sketch arena (-1: none)
  int n, m, r, W;
  int tab_off;        // offset into the hash-table arena (-1: none)
  int cnt_off;        // offset into the counts arena (-1: none)
  int q_rows;         // rows per CTA row-block in the Q = M^T P kernel
  int q_atomic;       // 1 if several CTAs (or several records) accumulate into the same Q block
  int src;            // 0: the matrix lives in the gradient bucket, 1: in the auxiliary buffer
  int Wp;             // row pitch of the sketch block in floats (W rounded up so that TMA can address it)
  long long qpk_off;  // packed copy of the (m x r) block for the tensor-core kernel (floats), see conef_pack_small
  long long ppk_off;  // packed copy of the (n x r) block
  // Folded view for matrices whose row pitch is not a multiple of 16 bytes (m % 4 != 0), which a
  // tensor map cannot describe: `fold` consecutive rows are read as ONE row of fold * m elements
  // (pitch then a multiple of 16 bytes), i.e. the same memory as an (n / fold) x (fold * m) matrix.
  //   P = M Q   : (n/f x f m)(f m x f r) with the block-diagonal operand diag(Q, .., Q) gives the
  //               (n/f x f r) result whose memory IS the (n x r) block P.
  //   Q = M^T P : (f m x n/f)(n/f x f r) with P read as (n/f x f r); output row b m + j holds in its
  //               columns [b r, (b+1) r) one part of Q[j, :]; the f parts are added up.
  // fold <= 1: no folding.  With fold > 1 the packed block at qpk_off is that block-diagonal operand
  // (f m rows) and ppk_fold_off the (n/f x f r) packing of P (ppk_off keeps the plain one).
  long long ppk_fold_off;
  int fold;
  // Block layout of the hash (columns hashed in aligned groups of 32, see k_psgd_decompress_blk): offset,
  // inside the hash-table arena, of the matrix's groups regrouped by cell block; -1: per-element hash.
  int cb_off;
} ConefMat;

// One small-factor correction (see conef_lowrank_correct): offsets in floats into the four
// base pointers given at launch.
typedef struct ConefCorr {
  long long t_off;          // T (rows_t x c1)
  long long x_off[2];       // X_t (rows_t x c2[t])
  long long l_off[2];       // L_t (rows_l x c2[t])
  long long r_off[2];       // Rm_t (rows_l x c1)
  int rows_t, rows_l, c1, nterms;
  int c2[2];
} ConefCorr;

// A contiguous run of elements of the bucket (one uncompressed tensor, or the
// selected part of a random block) and where it sits in a staging buffer.
typedef struct ConefSeg {
  long long src_off;  // offset inside the bucket
  long long dst_off;  // offset inside the staging buffer
  long long len;
} ConefSeg;

// One tensor handled by the random-block kernels, viewed as (n x m).
typedef struct ConefBlk {
  long long g_off;    // tensor start inside the bucket
  long long numel;
  long long start;    // first selected flat index
  long long block;    // number of selected elements (wraps around to index 0)
  long long stage_off;// offset of the block inside the staging buffer
  long long sk_off;   // sketch arena offset, or offset into the dense / quantised error arena
  int n, m, W;
  int tab_off, cnt_off;
  int scale_off;      // first scale slot of this tensor in the 8-bit store's scale array
  int cb_off;         // block layout of the hash: offset of the regrouped records in the table arena (-1: none)
  int pad_;
} ConefBlk;

enum { CONEF_EF_NONE = 0, CONEF_EF_DENSE = 1, CONEF_EF_SKETCH = 2, CONEF_EF_QUANT8 = 3 };

// Work that rides along with an orthogonalisation (conef_orthogonalize_fused), so that a bucket's
// pipeline needs no separate launches for it.  All members may be zero / NULL.
typedef struct ConefOrthExtra {
  // Two regions cleared by the Gram kernel's CTAs (with world > 1: after the flag wait, i.e. once
  // every peer is known to have finished reading them).
  float* zero0;  long long zero0_n;
  float* zero1;  long long zero1_n;
  // Uncompressed tensors, handled by spare CTAs of the Gram kernel.
  // seg_mode 1: staging[e] = bucket[...] (+ dense error, which then keeps the local value)
  // seg_mode 2: bucket[...] = seg_scale * sum over peers of peer_staging[p][e] (after the flag wait)
  int seg_mode, nsegs;
  const ConefSeg* segs;
  long long seg_total;
  float* bucket;
  float* dense_err;
  float* staging;
  const float* const* peer_staging;
  float seg_scale;
  // which == 1 only: the last pass adds alpha * s_j * Q[j, :] to cell h_j of the sketch record's
  // small operand Z = alpha H^T Q, directly in the packed layout the tensor-core kernel reads
  // (record nm + i describes the sketch of matrix i; `packed` must be given; the Z part of the
  // packed buffer must be one of the zeroed regions).
  float alpha;
  int nm;
  const int32_t* tables;
  // With `bar` (two device words, zero once) and `max_rank` (largest r among the records) the whole
  // orthogonalisation runs as one launch whose CTAs meet at two barriers, when the device can hold
  // all of them at once; otherwise, and when either is zero, as three launches.
  uint32_t* bar;
  int max_rank;
  // With `cl_list` (cl_nmat device entries {record, unused}: the records whose blocks the tile list covers)
  // and `cl_max_rows` (an upper bound of their row counts) every block is orthogonalised by one
  // thread-block cluster of eight CTAs that keep the block's rows in shared memory, exchange Gram
  // partials through distributed shared memory and meet at the cluster barrier; taken when a CTA's
  // share of the largest block fits in shared memory, before the one-launch form above.
  int cl_nmat;
  const int2* cl_list;
  int cl_max_rows;
  int pad_;
} ConefOrthExtra;

const char* conef_last_error(void);
int conef_version(void);
int conef_mat_size(void);       // sizeof(ConefMat), so that a binding can verify its mirror of the layout

// ---- count sketch (sketch.cu) ---------------------------------------------
// layout 0: per-element hash of the reference; 1: block layout (see conef_cell in common.cuh)
int conef_build_hash_table(int32_t* table, int32_t* counts, int D, int W,
                           int a, int b, int sa, int sb, int layout, cudaStream_t stream);
int conef_sketch_query(float* mat, const void* cs, int cs_is_half, const int32_t* table,
                       int N, int D, int W, float alpha, cudaStream_t stream);
int conef_sketch_update(const float* vec, void* cs, int cs_is_half, const int32_t* table,
                        const int32_t* counts, int N, int D, int W, float beta,
                        cudaStream_t stream);
int conef_sketch3_query(float* mat, const float* cs0, const float* cs1, const float* cs2,
                        const int32_t* t0, const int32_t* t1, const int32_t* t2,
                        int N, int D, int W, float alpha, cudaStream_t stream);
int conef_sketch3_update(const float* vec, float* cs0, float* cs1, float* cs2,
                         const int32_t* t0, const int32_t* t1, const int32_t* t2,
                         int N, int D, int W, float beta, cudaStream_t stream);

// ---- grouped PowerSGD pipeline, SIMT (powersgd.cu) --------------------------
// P_i (+)= A_i Q_i for every record: A_i is a matrix of the bucket (src 0) or of the
// auxiliary buffer (src 1: a sketch (n x W) or a dense error matrix).  With atomic_out
// the results are added to P (several records feed the same block), which the caller zeroed.
int conef_psgd_p(const ConefMat* mats, const int2* tiles, int ntiles, const float* bucket,
                 const float* aux, const float* Q, float* P, int atomic_out, int max_rank,
                 cudaStream_t stream);
// Orthonormalise the (rows x r) blocks of a flat buffer: which = 0 the P blocks (n x r),
// which = 1 the Q blocks (m x r).  Row-parallel Gram-Schmidt through the Gram matrix, applied
// twice (csrc/orth.cu).  tiles: int2 {record, chunk of 512 rows}.  With world > 1 each chunk
// first waits (bounded) until every peer has published `epoch` in flags[peer] and sums the
// peers' buffers (peer_bufs[0..world)) into `buf`; status[0] becomes non-zero when a wait gives up.
// packed (nullable): also write the result in the tensor-core operand layout with packed_np columns.
// gram: scratch of 2 * ntiles * 1024 floats.  The result depends only on the input bits (fixed
// summation order), so ranks that start from the same reduced P end with the same factors.
int conef_orthogonalize_packed(const ConefMat* mats, const int2* tiles, int ntiles, int nrecords,
                               int which, float* buf, float eps, const float* const* peer_bufs,
                               const uint32_t* flags, int world, uint32_t epoch, int* status,
                               long long spin_limit, float* packed, int packed_np, float* gram,
                               cudaStream_t stream);
int conef_psgd_q(const ConefMat* mats, const int2* tiles, int ntiles, const float* bucket,
                 const float* aux, const float* P, float* Q, int max_rank, cudaStream_t stream);
// M_hat = P Q^T written into the bucket.  M = G + remembered error is formed on the fly
// (alpha * unsketch(S) or the dense buffer); the residual M - M_hat goes to the error
// store selected by ef_mode (dense buffer, or count sketch with decay beta).
// smem_bytes = rows_per_cta * max W * 4 in sketch mode, else 0.
// In sketch mode the first nblk_tiles tiles belong to matrices whose hash has the block layout
// (cb_off >= 0): they run on the atomics-free kernel that walks the columns cell block by cell block.
// Such a tile is (matrix, chunk of 8 units); a unit is (rbu consecutive row blocks, cell block), rbu in
// 1..4, and 1 regardless for matrices with more than 32 windows; a matrix has
// ceil(ceil(n / rows_per_cta) / rbu) * (W / 32) units.
int conef_psgd_decompress(const ConefMat* mats, const int2* tiles, int ntiles, int nblk_tiles, int rbu,
                          int rows_per_cta,
                          float* bucket, const float* P, const float* Q, float q_scale,
                          float* sketch, const int32_t* tables, const int32_t* counts,
                          float* dense_err, float alpha, float beta, int ef_mode, int max_rank,
                          size_t smem_bytes, int* status, cudaStream_t stream);
// status: device word that receives CONEF_STATUS_MBAR_TIMEOUT when a bounded wait of the bulk-copy
// ring runs out (NULL: the ring is filled with cp.async, which needs no waits on barriers).
// Sparse sign matrix H of the sketch applied to the small factors (see csrc/sketch.cu):
// unproject = 0: Z_i += scale * H_i^T Q_i ; unproject = 1: Q_i += scale * H_i Y_i.
// Record nmats + i describes the sketch of matrix i; its q_off is where Z_i / Y_i live.
int conef_sketch_project(const ConefMat* mats, int nmats, int max_cols, const int32_t* tables,
                         float* qz, float scale, int unproject, cudaStream_t stream);
// All-reduce of the Q blocks over peer memory fused with the sketch term's un-projection:
// out Q_i[j, :] = scale * sum_p ( Q_p,i[j, :] + alpha s_j Y_p,i[h_j, :] ), every peer buffer laid out
// [Q blocks | Y blocks] like `out`'s own buffer.  Waits (bounded) until my_flags[0..world) reached
// `epoch` (+ *epoch_base); world == 1: no wait, peer_bufs[0] is local.  tables == NULL: plain sum.
int conef_reduce_q(const ConefMat* mats, int nmats, int max_cols, const int32_t* tables, float* out,
                   const float* const* peer_bufs, const uint32_t* my_flags, int world, uint32_t epoch,
                   float alpha, float scale, int* status, long long spin_limit, const uint32_t* epoch_base,
                   cudaStream_t stream);
// Per matrix: T (rows_t x c1) += sum over up to two terms of coef_t * X_t (rows_t x c2_t) * (L_t^T Rm_t).
// Used by the low-rank error store, whose factors enter PowerSGD's products as small corrections.
// reduce_tiles chunk rows_l, apply_tiles chunk rows_t (int2 {matrix, chunk of 512 rows});
// cbuf: scratch of nmats * 2 * 1024 floats.
int conef_lowrank_correct(const ConefCorr* table, int nmats, const int2* reduce_tiles, int n_reduce,
                          const int2* apply_tiles, int n_apply, float* T, const float* X0, const float* L0,
                          const float* R0, float coef0, const float* X1, const float* L1, const float* R1,
                          float coef1, float* cbuf, cudaStream_t stream);
// Philox-keyed standard normal fill: element e of the buffer depends only on
// (seed, e), so every rank generates the same Q without communication.
int conef_fill_normal(float* buf, long long numel, uint64_t seed, cudaStream_t stream);

// ---- tcgen05 / TMEM / TMA tiles (powersgd_tc.cu) ----------------------------
int conef_tc_supported(void);
// Host side: two 128-byte tensor maps per matrix into maps_out (256 bytes per matrix);
// ok[i] = 0 when matrix i cannot be addressed by TMA (base not 16-byte aligned or row
// pitch not a multiple of 16 bytes).
int conef_tc_encode_maps(const ConefMat* host_mats, int nmats, const float* bucket_dev,
                         const float* aux_dev, void* maps_out_256B_each, unsigned char* ok);
// mode 0: P = M Q (small operand Q, output P).  mode 1: Q = M^T P (small operand P, output Q).
// tiles: int4 records {matrix | atomic << 30, first output row, first K index, K extent}.
// small_packed: the small operands in the tensor-core operand layout (conef_pack_small).
int conef_psgd_tc(int mode, const ConefMat* mats, const void* maps, const void* tiles, int ntiles,
                  const float* small_packed, float* out_base, int max_rank, int* status,
                  cudaStream_t stream);
// The same, and the CTA that finishes last publishes `epoch` (+ *epoch_base when given) in slot
// `rank` of every peer's flag array (done: a device counter, zero between launches).  With
// done == NULL or world == 1 nothing is published.
int conef_psgd_tc_signal(int mode, const ConefMat* mats, const void* maps, const void* tiles, int ntiles,
                         const float* small_packed, float* out_base, int max_rank, int* status,
                         uint32_t* done, uint32_t* const* peer_flags, int world, int rank, uint32_t epoch,
                         const uint32_t* epoch_base, cudaStream_t stream);
// Copy the (rows x r) blocks of `src` (which = 0: P blocks, 1: Q blocks) into the layout the
// tensor-core kernel reads with one bulk copy per stage: K-major 8x4 core matrices, r padded
// with zeros to NP = 16 (max_rank <= 16) or 32 columns, rows padded to a multiple of 32.
// Pad cells are never written: `dst` must be zero-initialised once.
int conef_pack_small(const ConefMat* mats, int nrec, int which, const float* src, float* dst,
                     int max_rank, cudaStream_t stream);

// ---- grouped magnitude top-k (topk.cu) -----------------------------------------
// For each of the first nmats records: keep the max(1, int(0.5 * ratio * n * m)) largest-magnitude
// entries of the (n x m) matrix at err + g_off and zero the rest (entries tying with the k-th
// magnitude are all kept).  tiles: int2 {matrix, chunk of conef_topk_chunk() elements}.
// scratch: nmats * (2048 + 2) 32-bit words, zeroed once by the caller.
int conef_topk_keep(const ConefMat* mats, int nmats, const int2* tiles, int ntiles, float* err,
                    float ratio, uint32_t* scratch, cudaStream_t stream);
int conef_topk_chunk(void);

// ---- segments, random blocks, quantised error (blocks.cu) -------------------
int conef_gather_segments(const ConefSeg* segs, int nsegs, const float* bucket,
                          const float* dense_err, float* staging, long long total,
                          cudaStream_t stream);
// bucket[seg] = scale * sum_peers staging_peer[seg]; with dense_err != NULL the
// pre-reduction local value minus the result is stored as the new error.
int conef_scatter_segments(const ConefSeg* segs, int nsegs, float* bucket,
                           const float* const* peer_staging, int world, const float* local_staging,
                           float scale, float* dense_err, long long total, cudaStream_t stream);
// Count-sketch mode: the first nblk_tiles tiles belong to tensors on the block layout of the hash
// (cb_off >= 0) and are chunks of eight (block of 8 rows, cell block) units; the others are
// (tensor, block of rows_per_cta rows).
int conef_randblock_gather(const ConefBlk* blks, const int2* tiles, int ntiles, int nblk_tiles, int rows_per_cta,
                           float* bucket, float* staging, float gather_scale,
                           float* sketch, const int32_t* tables, const int32_t* counts,
                           float* dense_err, int8_t* qcodes, float* qscales,
                           float alpha, float beta, int ef_mode, size_t smem_bytes,
                           cudaStream_t stream);
// The same gather with the uncompressed tensors copied into staging_unc by spare CTAs and, with
// done != NULL and world > 1, the CTA that finishes last publishing `epoch` (+ *epoch_base) in slot
// `rank` of every peer's flag array.
int conef_randblock_gather_ex(const ConefBlk* blks, const int2* tiles, int ntiles, int nblk_tiles, int rows_per_cta,
                              float* bucket, float* staging, float gather_scale, float* sketch,
                              const int32_t* tables, const int32_t* counts, float* dense_err, int8_t* qcodes,
                              float* qscales, float alpha, float beta, int ef_mode, size_t smem_bytes,
                              const ConefSeg* segs, int nsegs, long long total_unc, float* staging_unc,
                              uint32_t* done, uint32_t* const* peer_flags, int world, int rank, uint32_t epoch,
                              const uint32_t* epoch_base, cudaStream_t stream);
// One launch: bounded wait for `epoch` (world > 1), sum of the peers' staged values in rank order,
// averages written into the bucket (uncompressed tensors and blocks).  two_shot: every rank sums its
// 1/world slice of the blocks, stores it into every peer's `reduced` buffer (peer_red), publishes
// epoch + 1, waits for the peers' and scatters from my_red.
int conef_randblock_reduce_scatter(const ConefBlk* blks, int nblks, const ConefSeg* segs, int nsegs,
                                   long long total_unc, long long total_blk, float* bucket,
                                   const float* const* peer_unc, const float* const* peer_blk,
                                   float* const* peer_red, const float* my_red, uint32_t* const* peer_flags,
                                   const uint32_t* my_flags, int world, int rank, uint32_t epoch,
                                   const uint32_t* epoch_base, float scale, int two_shot, uint32_t* done,
                                   int* status, long long spin_limit, cudaStream_t stream);
int conef_randblock_scatter(const ConefBlk* blks, int nblks, float* bucket,
                            const float* const* peer_staging, int world,
                            const float* local_staging, float scale, long long total_block,
                            cudaStream_t stream);
int conef_quant8_query(float* x, const int8_t* codes, const float* scales, long long numel,
                       float alpha, cudaStream_t stream);
int conef_quant8_update(const float* v, int8_t* codes, float* scales, long long numel,
                        float beta, cudaStream_t stream);

// ---- in-kernel collectives over peer memory (symm.cu) -----------------------
// Publish `epoch` into slot `rank` of every peer's flag array.
int conef_signal_peers(uint32_t* const* peer_flags, int world, int rank, uint32_t epoch,
                       cudaStream_t stream);
// out[i] = scale * sum_p peer_bufs[p][i] after a bounded wait on flags.
int conef_allreduce_oneshot(float* out, const float* const* peer_bufs, uint32_t* const* peer_flags,
                            const uint32_t* my_flags, int world, int rank, uint32_t epoch,
                            long long numel, float scale, int* status, long long spin_limit,
                            cudaStream_t stream);
int conef_wait_flags(const uint32_t* my_flags, int world, uint32_t epoch, int* status,
                     long long spin_limit, cudaStream_t stream);
// Variants with `epoch_base` (nullable device word added to `epoch` on the device): a captured
// launch replayed from a CUDA graph gets a fresh epoch each time without new kernel arguments.
int conef_signal_peers_ex(uint32_t* const* peer_flags, int world, int rank, uint32_t epoch,
                          const uint32_t* epoch_base, cudaStream_t stream);
int conef_allreduce_oneshot_ex(float* out, const float* const* peer_bufs, uint32_t* const* peer_flags,
                               const uint32_t* my_flags, int world, int rank, uint32_t epoch,
                               long long numel, float scale, int* status, long long spin_limit,
                               const uint32_t* epoch_base, cudaStream_t stream);
int conef_wait_flags_ex(const uint32_t* my_flags, int world, uint32_t epoch, int* status,
                        long long spin_limit, const uint32_t* epoch_base, cudaStream_t stream);
int conef_orthogonalize_packed_ex(const ConefMat* mats, const int2* tiles, int ntiles, int nrecords,
                                  int which, float* buf, float eps, const float* const* peer_bufs,
                                  const uint32_t* flags, int world, uint32_t epoch, int* status,
                                  long long spin_limit, float* packed, int packed_np, float* gram,
                                  const uint32_t* epoch_base, cudaStream_t stream);
// The same with the ride-along work of ConefOrthExtra.  With peer_bufs given and world == 1 the
// input is read from peer_bufs[0] (no flags) and the result written to buf.
int conef_orthogonalize_fused(const ConefMat* mats, const int2* tiles, int ntiles, int which, float* buf,
                              float eps, const float* const* peer_bufs, const uint32_t* flags, int world,
                              uint32_t epoch, int* status, long long spin_limit, float* packed,
                              int packed_np, float* gram, const uint32_t* epoch_base,
                              const ConefOrthExtra* extra, cudaStream_t stream);
// Kernels enqueued by the calling thread's most recent conef_orthogonalize_* call.
int conef_orth_last_launches(void);
// *word = value (add = 0) or *word += value (add = 1), in stream order.
int conef_epoch_word(uint32_t* word, uint32_t value, int add, cudaStream_t stream);
int conef_ipc_get_handle(void* dev_ptr, void* handle_out_64B);
int conef_ipc_open_handle(const void* handle_64B, void** dev_ptr_out);
int conef_ipc_close_handle(void* dev_ptr);

// ---- multi-tensor LAMB (lamb.cu) --------------------------------------------
typedef struct ConefLambTensor {
  float* p;          // parameter (fp32)
  float* g;          // gradient on entry; overwritten with the LAMB update direction
  float* m;          // first moment
  float* v;          // second moment
  long long numel;
  float weight_decay;
  int pad;
} ConefLambTensor;
// norms: scratch of 1 + 2*ntensors floats ([0] squared global gradient norm,
// [1+2t] squared parameter norm, [2+2t] squared update norm of tensor t).
int conef_lamb_step(const ConefLambTensor* tensors, int ntensors, const int2* chunks, int nchunks,
                    int chunk_elems, float* norms, float lr, float beta1, float beta2, float eps,
                    int step, int bias_correction, float grad_scale, float max_grad_norm,
                    cudaStream_t stream);

// Multi-tensor SGD with momentum (torch.optim.SGD semantics; weight decay per tensor from the table, `v` unused;
// first != 0: the momentum buffers are initialised with the gradient).
int conef_sgd_step(const ConefLambTensor* tensors, int ntensors, const int2* chunks, int nchunks, int chunk_elems,
                   float lr, float momentum, float dampening, int nesterov, int first, cudaStream_t stream);

// ---- column sums (colsum.cu) -------------------------------------------------
// out[c] = sum over rows of x[row, c] for a row-major (rows x cols) matrix: the bias gradient of a convolution
// whose output gradient lies in channels-last memory.  dtype: 0 fp32, 1 bf16, 2 fp16.  partial: scratch of
// nparts * cols floats (one partial row per CTA, added up in CTA order by a second kernel).  Returns 2 for
// inputs it does not take (cols % 8 != 0, cols > 2048, x not 16-byte aligned).
int conef_colsum(const void* x, int dtype, long long rows, int cols, float* partial, int nparts, float* out,
                 cudaStream_t stream);
// Batch-norm statistics of the same kind of matrix: mean and 1 / sqrt(biased variance + eps) per column from
// shifted sums, plus the momentum update of the running statistics (NULL: none).  partial: nparts * 2 * cols floats.
int conef_colstats(const void* x, int dtype, long long rows, int cols, float eps, float momentum, float* partial,
                   int nparts, float* mean, float* invstd, float* running_mean, float* running_var,
                   cudaStream_t stream);
// The two sums of the batch-norm backward pass: sum_dy = sum dy, sum_dy_xmu = sum dy (x - mean); grad_weight
// (= sum_dy_xmu * invstd) and grad_bias (= sum_dy) when given.  dy and x share dtype and layout.
int conef_coldot(const void* dy, const void* x, int dtype, long long rows, int cols, const float* mean,
                 const float* invstd, float* partial, int nparts, float* sum_dy, float* sum_dy_xmu,
                 float* grad_weight, float* grad_bias, cudaStream_t stream);
// Elementwise passes of batch norm, optionally fused with the ReLU behind it (relu != 0):
//   conef_bn_apply          y = relu?((x - mean) invstd weight + bias)
//   conef_coldot_relu       conef_coldot with dy masked where that ReLU is inactive
//   conef_bn_backward_apply gx = (gy - sum_dy / n - (x - mean) invstd^2 sum_dy_xmu / n) invstd weight (gy masked likewise)
// nparts CTAs split the rows; weight / bias may be NULL (1 and 0).
// Weight and bias gradients of a layer norm along the rows of a (rows x cols) activation:
// dgamma[c] = sum_rows dy (x - mean[row]) rstd[row], dbeta[c] = sum_rows dy.  partial: nparts * 2 * cols floats.
int conef_ln_wgrad(const void* dy, const void* x, int dtype, long long rows, int cols, const float* mean,
                   const float* rstd, float* partial, int nparts, float* dgamma, float* dbeta, cudaStream_t stream);
// dst (bf16) = src (fp32), n elements; both 16-byte aligned
int conef_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream);
// y[row, c] += bias[c] in place (the bias of a convolution with a channels-last output)
int conef_bias_add(void* y, int dtype, long long rows, int cols, const float* bias, int nparts, cudaStream_t stream);
int conef_bn_apply(const void* x, void* y, int dtype, long long rows, int cols, const float* mean, const float* invstd,
                   const float* weight, const float* bias, int relu, int nparts, cudaStream_t stream);
int conef_coldot_relu(const void* dy, const void* x, int dtype, long long rows, int cols, const float* mean,
                      const float* invstd, const float* weight, const float* bias, float* partial, int nparts,
                      float* sum_dy, float* sum_dy_xmu, float* grad_weight, float* grad_bias, cudaStream_t stream);
int conef_bn_backward_apply(const void* gy, const void* x, void* gx, int dtype, long long rows, int cols,
                            const float* mean, const float* invstd, const float* weight, const float* bias,
                            const float* sum_dy, const float* sum_dy_xmu, int relu, int nparts, cudaStream_t stream);

// ---- host implementations (cpu_ops.cu) --------------------------------------
void conef_cpu_hash_table(int32_t* table, int32_t* counts, int D, int W, int a, int b, int sa, int sb, int layout);
void conef_cpu_sketch_query(float* mat, const float* cs, const int32_t* table, int N, int D, int W, float alpha);
void conef_cpu_sketch_update(const float* vec, float* cs, const int32_t* table, const int32_t* counts,
                             int N, int D, int W, float beta);
void conef_cpu_gram_schmidt(float* mat, int rows, int cols, float eps);

#ifdef __cplusplus
}
#endif
