// Native per-bucket executor of the PowerSGD family: one host call enqueues the whole
// compression pipeline of a bucket (about a dozen grouped launches plus memsets and small
// copies) on a stream.  The reference drives its pipeline from Python futures with ~10^4 tiny
// launches and one device synchronisation per bucket (communication/powerSGD_hook.py:394-580);
// here even the Python-side launch loop is gone from the hot path: the plan is filled once per
// bucket layout and only a few per-step fields change.
#pragma once
#include "conef.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ConefTileList {
  const void* tiles;
  int n;
  int pad;
} ConefTileList;

typedef struct ConefQSet {       // tiles of the Q = M^T P pass for one subset of records
  ConefTileList tc;              // tensor-core tiles (int4)
  ConefTileList simt;            // SIMT tiles (int2)
} ConefQSet;

typedef struct ConefPsgdPlan {
  // ---- static: filled once per bucket layout -------------------------------------------
  const ConefMat* mats;
  int nrec, nm, max_rank, np_cols, max_cols;
  int unbiased;                  // random-projection compressor: no Gram-Schmidt, no Q pass, P averaged
  int ef_mode;                   // CONEF_EF_*
  int lowrank;                   // low-rank error store (records nm.. multiply by the error factors)
  int use_tc, p_zero, q_zero;
  const int32_t* tables;
  const int32_t* counts;
  float* sketch;
  float* dense_err;
  const float* aux;              // error buffer read by the src = 1 records (sketch arena or dense error)
  float* qz;  long long total_q, total_z;     // [Q | Z or V]
  float* pu;  long long total_p, total_u;     // [P | U']
  float* u_old;
  float* qz2;
  float* qpk;
  float* ppk;
  const ConefSeg* segs;  int nsegs, orth_max_rows;  long long total_unc;      // orth_max_rows: most rows of any P or Q block
                                                                             // (0: no cluster form of the Gram-Schmidt kernel)
  float* staging;
  const void* tc_maps;
  ConefTileList tc_p, simt_p;
  ConefQSet qset_all, qset_grad, qset_err;
  ConefTileList d_tiles;  int d_rows, d_nblk;  size_t d_smem;      // d_nblk: leading tiles on the block layout
  ConefTileList orth_q, orth_p, orth_u, chunks_n, chunks_m;
  float* gram;
  float* cbuf;
  const ConefCorr* corr_p;
  const ConefCorr* corr_q;
  const ConefCorr* corr_u;
  const ConefCorr* corr_v;
  int* status;
  // ---- peer memory (world > 1 with symmetric buffers) -------------------------------------
  int world, rank, has_symm, d_rbu;      // d_rbu: row blocks per unit of the block-layout decompress
  uint32_t* const* peer_flags;   // device array [world] of the peers' flag arrays
  const uint32_t* my_flags;
  const float* const* peer_stage[2];   // per slot: device arrays [world] of region pointers
  const float* const* peer_p[2];
  const float* const* peer_q[2];
  float* local_stage[2];
  float* local_p[2];
  float* local_q[2];
  long long spin_limit;
  // ---- per step ------------------------------------------------------------------------------
  float* work;                   // the bucket (or the padded square of the batched variant)
  int slot;
  int fresh;                     // draw a new random Q from `seed`
  unsigned long long seed;
  unsigned int epoch;            // in/out: advanced by one per in-kernel collective
  float alpha, beta, eps;
  int launched;                  // out: kernels enqueued by the call
  // ---- CUDA-graph replay (conef_psgd_step) ------------------------------------------------------
  int use_graph;                 // 1: capture the pipeline once per slot and replay it
  uint32_t* epoch_word;          // device word holding the epoch base of replayed launches
  unsigned int epoch_shadow;     // what the host believes *epoch_word holds
  int graph_runs[2];             // direct runs done per slot before the capture
  void* graph_exec[2];           // cudaGraphExec_t per slot
  int graph_launched[2];         // kernels inside each captured graph
  int graph_ncoll[2];            // in-kernel collectives inside each captured graph
  float* key_work;               // what the graphs were captured with
  float key_alpha, key_beta, key_eps;
  int graph_replays;             // out: number of graph launches so far
  // ---- top-k error store (dense error buffer pruned after every step) ---------------------------
  int topk;                      // 1: dense_err holds the matrices' errors only (no error for the
                                 //    uncompressed tensors) and is pruned to its largest entries
  float topk_ratio;
  ConefTileList topk_tiles;
  uint32_t* topk_scratch;
  // ---- fused pipeline (ten launches per bucket and step) -------------------------------------------
  int fused;                     // 1: run_fused (see executor.cu); needs tensor-core tiles in both products,
                                 //    no low-rank store, not the unbiased variant, and slot buffers
  int has_slots;                 // local_* / peer_* are set (symmetric memory, or plain local buffers with
                                 //    one-entry pointer tables when world == 1); they start zeroed
  uint32_t* done_word;           // device counter of the tile kernel's finished CTAs (zero between launches)
  float* zpk;  long long zpk_n;  // packed small operands of the sketch records inside qpk
  int one_launch_orth;           // 1: orthogonalisations as one launch with two CTA barriers (done_word[1..2])
  int wait_kernel;               // 1 (world > 1): a one-CTA kernel waits for the peers' epoch ahead of each consumer
  int orth_rows_q, orth_rows_p, orth_rows_u, pad3;   // most rows of a block in each Gram-Schmidt tile list
} ConefPsgdPlan;

// ---- random-block family ---------------------------------------------------------------------------
typedef struct ConefRandblockPlan {
  // static
  const ConefBlk* blks;  int nblks, rows_per_cta;      // the block table is re-uploaded every step (new offsets)
  ConefTileList tiles;
  const ConefSeg* segs;  int nsegs, ef_mode;
  long long total_unc, total_block;
  float* staging_unc;  float* staging_blk;              // local staging (no peer memory)
  float* sketch;  const int32_t* tables;  const int32_t* counts;
  float* dense_err;  int8_t* qcodes;  float* qscales;
  size_t smem;
  int* status;
  int world, rank, has_symm, unbiased;
  uint32_t* const* peer_flags;  const uint32_t* my_flags;
  const float* const* peer_unc[2];  const float* const* peer_blk[2];
  float* local_unc[2];  float* local_blk[2];
  long long spin_limit;
  // per step
  float* work;  int slot, nblk_tiles;      // nblk_tiles: leading tiles of tensors on the block layout of the hash
  unsigned int epoch;  float alpha, beta;
  int launched;
  // ---- two-launch form: gather (+ segments, publishes the epoch) and wait + reduce + scatter ----
  int has_slots;                 // local_* / peer_* set (symmetric memory, or local buffers when world == 1)
  int two_shot;                  // 1: blocks reduced in two shots through the `reduced` buffers
  float* const* peer_red[2];     // per slot: device arrays [world] of the peers' `reduced` buffers
  const float* local_red[2];
  uint32_t* done_word;           // device counter of finished CTAs (zero between launches)
} ConefRandblockPlan;

// With has_slots: two launches (see csrc/blocks.cu).  Otherwise:
// Gather (block -> staging, error update), reduction over peer memory (bounded wait), scatter.
// phases: 1 = gather, 2 = scatter; without peer memory and world > 1 the caller all-reduces the two
// staging buffers between the phases.
int conef_randblock_run(ConefRandblockPlan* plan, int phases, cudaStream_t stream);
int conef_randblock_plan_size(void);

enum { CONEF_PHASE_P = 1, CONEF_PHASE_Q = 2, CONEF_PHASE_D = 4, CONEF_PHASE_ALL = 7 };

// phases: P = up to and including P = G Q (+ error terms);  Q = reduction of P (peer memory only),
// Gram-Schmidt, scatter of the uncompressed tensors, Q = G^T P;  D = reduction of Q (peer memory
// only), refresh of the low-rank factors, decompress + error update.  Without symmetric buffers and
// world > 1 the caller runs the phases one by one and all-reduces P (after P) and Q (after Q) itself.
int conef_psgd_run(ConefPsgdPlan* plan, int phases, cudaStream_t stream);
int conef_psgd_plan_size(void);
// The whole pipeline for one step (all phases; needs world == 1 or peer memory).  With
// plan->use_graph, steps that draw no new random Q are captured into a CUDA graph per buffer slot
// after two direct runs and replayed afterwards: one graph launch instead of ~20 kernel launches.
// A change of the bucket address or of alpha / beta / eps drops the graphs.  If a capture fails the
// plan falls back to direct launches for good.
int conef_psgd_step(ConefPsgdPlan* plan, cudaStream_t stream);
// Destroy the captured graphs of a plan.
int conef_psgd_plan_release(ConefPsgdPlan* plan);

#ifdef __cplusplus
}
#endif
