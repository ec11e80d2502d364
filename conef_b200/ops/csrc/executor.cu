// Native per-bucket executor of the PowerSGD family (see executor.h).
#include "executor.h"
#include <string.h>

#define RUN(call)                      \
  do {                                 \
    int rc_ = (call);                  \
    if (rc_ != 0) return rc_;          \
    ++plan->launched;                  \
  } while (0)

#define CUDA_OK(call)                                   \
  do {                                                  \
    cudaError_t e_ = (call);                            \
    if (e_ != cudaSuccess) return (int)e_;              \
  } while (0)

namespace {

inline int zero_floats(float* p, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  return (int)cudaMemsetAsync(p, 0, (size_t)n * sizeof(float), s);
}

inline int copy_floats(float* dst, const float* src, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)n * sizeof(float), cudaMemcpyDeviceToDevice, s);
}

// A tile list's `pad` entries behind its `n` tiles name the records it covers: the cluster form of the
// Gram-Schmidt kernel goes by record, not by chunk of rows.
inline void set_cluster_list(const ConefPsgdPlan* plan, const ConefTileList& tl, int max_rows, ConefOrthExtra& X) {
  if (plan->one_launch_orth && plan->orth_max_rows > 0 && tl.pad > 0 && max_rows > 0) {
    X.cl_list = (const int2*)tl.tiles + tl.n;
    X.cl_nmat = tl.pad;
    X.cl_max_rows = max_rows;
  }
}

int orth(ConefPsgdPlan* plan, int which, const ConefTileList& tl, float* buf, float eps,
         const float* const* peers, const uint32_t* flags, int world, uint32_t epoch, bool packed,
         cudaStream_t s, const uint32_t* eb = nullptr) {
  if (!tl.n) return 0;
  float* pk = (packed && plan->use_tc) ? (which == 0 ? plan->ppk : plan->qpk) : nullptr;
  ConefOrthExtra X;
  memset(&X, 0, sizeof(X));
  X.bar = (plan->one_launch_orth && plan->done_word) ? plan->done_word + 1 : nullptr;    // one launch when it fits
  X.max_rank = plan->max_rank;
  set_cluster_list(plan, tl, &tl == &plan->orth_q ? plan->orth_rows_q : &tl == &plan->orth_p ? plan->orth_rows_p
                                                                                             : plan->orth_rows_u, X);
  RUN(conef_orthogonalize_fused(plan->mats, (const int2*)tl.tiles, tl.n, which, buf, eps,
                                world > 1 ? peers : nullptr, flags, world, epoch, plan->status,
                                world > 1 ? plan->spin_limit : 0, pk, plan->np_cols, plan->gram, eb, &X, s));
  plan->launched += conef_orth_last_launches() - 1;
  return 0;
}

int launch_p(ConefPsgdPlan* plan, const float* aux, float* p_target, cudaStream_t s) {
  if (plan->use_tc && plan->tc_p.n) {
    RUN(conef_pack_small(plan->mats, plan->nrec, 1, plan->qz, plan->qpk, plan->max_rank, s));
    RUN(conef_psgd_tc(0, plan->mats, plan->tc_maps, plan->tc_p.tiles, plan->tc_p.n, plan->qpk,
                      p_target, plan->max_rank, plan->status, s));
  }
  if (plan->simt_p.n)
    RUN(conef_psgd_p(plan->mats, (const int2*)plan->simt_p.tiles, plan->simt_p.n, plan->work, aux,
                     plan->qz, p_target, plan->p_zero, plan->max_rank, s));
  return 0;
}

// The packed copy of the small operand is always current here: the Gram-Schmidt kernel writes it.
int launch_q(ConefPsgdPlan* plan, const ConefQSet& qs, const float* aux, const float* pmem,
             float* q_target, cudaStream_t s) {
  if (plan->use_tc && qs.tc.n)
    RUN(conef_psgd_tc(1, plan->mats, plan->tc_maps, qs.tc.tiles, qs.tc.n, plan->ppk, q_target,
                      plan->max_rank, plan->status, s));
  if (qs.simt.n)
    RUN(conef_psgd_q(plan->mats, (const int2*)qs.simt.tiles, qs.simt.n, plan->work, aux, pmem,
                     q_target, plan->max_rank, s));
  return 0;
}

struct Term { const float *x, *l, *r; float coef; };

int correct(ConefPsgdPlan* plan, const ConefCorr* table, bool over_n, float* T, Term t0, Term t1,
            cudaStream_t s) {
  const ConefTileList& red = over_n ? plan->chunks_n : plan->chunks_m;
  const ConefTileList& app = over_n ? plan->chunks_m : plan->chunks_n;
  RUN(conef_lowrank_correct(table, plan->nm, (const int2*)red.tiles, red.n, (const int2*)app.tiles,
                            app.n, T, t0.x, t0.l, t0.r, t0.coef, t1.x, t1.l, t1.r, t1.coef,
                            plan->cbuf, s));
  plan->launched += 1;      // a reduction and an application kernel
  return 0;
}

}  // namespace

#define OK(call)                       \
  do {                                 \
    int rc_ = (call);                  \
    if (rc_ != 0) return rc_;          \
  } while (0)

// The fused pipeline: ten launches per bucket and step (plus the SIMT kernels of matrices that TMA
// cannot address, and the top-k pruning).
//   P:  k_gram(Q) [+ clears the sketch records' packed operand, + gathers the uncompressed tensors]
//       k_qr_apply, k_qr_apply [final pass: writes Q packed, adds alpha H^T Q into the packed Z]
//       k_tc_skinny<P>  [last CTA publishes epoch 1 to the peers]
//   Q:  k_gram(P) [waits for epoch 1, sums the peers' P, clears the other slot's P and Q regions,
//                  spare CTAs sum the peers' staged tensors back into the bucket]
//       k_qr_apply, k_qr_apply [final pass writes P packed]
//       k_tc_skinny<Q>  [last CTA publishes epoch 2]
//   D:  k_reduce_q [waits for epoch 2, sums the peers' Q and un-projects the sketch term]
//       k_psgd_decompress
// The products accumulate with atomics into slot buffers that the Gram kernel of the following step
// clears, after its flag wait has shown that every peer is done reading them, so nothing is memset.
static int run_fused(ConefPsgdPlan* plan, int phases, cudaStream_t s, const uint32_t* eb, int* ncoll) {
  const uint32_t ebase = eb ? 0u : plan->epoch;
  const int nm = plan->nm, ws = plan->world, slot = plan->slot & 1;
  const bool peers = ws > 1;
  const bool sketch = plan->ef_mode == CONEF_EF_SKETCH;
  const bool fused_err = sketch || plan->ef_mode == CONEF_EF_DENSE;
  const float* aux = fused_err ? plan->aux : nullptr;
  const long long tq = plan->total_q, tz = plan->total_z, tp = plan->total_p, tu = plan->total_u;
  float* dense_err = plan->ef_mode == CONEF_EF_DENSE ? plan->dense_err : nullptr;
  float* seg_err = plan->topk ? nullptr : dense_err;
  float* p_target = plan->local_p[slot];
  float* q_target = plan->local_q[slot];
  const float inv_ws = 1.0f / (float)ws;
  const long long spin = peers ? plan->spin_limit : 0;
  uint32_t* const* pflags = peers ? plan->peer_flags : nullptr;

  if (phases & CONEF_PHASE_P) {
    if (plan->fresh) RUN(conef_fill_normal(plan->qz, tq, plan->seed, s));
    ConefOrthExtra X;
    memset(&X, 0, sizeof(X));
    X.bar = plan->one_launch_orth ? plan->done_word + 1 : nullptr;
    X.max_rank = plan->max_rank;
    set_cluster_list(plan, plan->orth_q, plan->orth_rows_q, X);
    if (sketch) { X.zero0 = plan->zpk; X.zero0_n = plan->zpk_n; X.tables = plan->tables; X.nm = nm; X.alpha = plan->alpha; }
    if (plan->total_unc) {
      X.seg_mode = 1; X.nsegs = plan->nsegs; X.segs = plan->segs; X.seg_total = plan->total_unc;
      X.bucket = plan->work; X.dense_err = seg_err; X.staging = plan->local_stage[slot];
    }
    RUN(conef_orthogonalize_fused(plan->mats, (const int2*)plan->orth_q.tiles, plan->orth_q.n, 1, plan->qz,
                                  plan->eps, nullptr, nullptr, 1, 0, plan->status, 0, plan->qpk, plan->np_cols,
                                  plan->gram, nullptr, &X, s));
    plan->launched += conef_orth_last_launches() - 1;
    if (plan->simt_p.n)
      RUN(conef_psgd_p(plan->mats, (const int2*)plan->simt_p.tiles, plan->simt_p.n, plan->work, aux, plan->qz,
                       p_target, 1, plan->max_rank, s));
    const uint32_t ep = ebase + (uint32_t)(++*ncoll);
    RUN(conef_psgd_tc_signal(0, plan->mats, plan->tc_maps, plan->tc_p.tiles, plan->tc_p.n, plan->qpk, p_target,
                             plan->max_rank, plan->status, plan->done_word, pflags, ws, plan->rank, ep, eb, s));
  }

  if (phases & CONEF_PHASE_Q) {
    // the epoch the P pass published: in this call, or in the previous one when the phases run one by one
    const uint32_t ep1 = ebase + (uint32_t)*ncoll;
    ConefOrthExtra X;
    memset(&X, 0, sizeof(X));
    // A one-CTA waiter first: when a peer is late, one CTA spins instead of every CTA of the next
    // kernel sitting on the SMs that this GPU's own backward pass could use; the waits inside the
    // consumers then pass at once.
    if (peers && plan->wait_kernel)
      RUN(conef_wait_flags_ex(plan->my_flags, ws, ep1, plan->status, spin, eb, s));
    X.bar = plan->one_launch_orth ? plan->done_word + 1 : nullptr;
    X.max_rank = plan->max_rank;
    set_cluster_list(plan, plan->orth_p, plan->orth_rows_p, X);
    X.zero0 = plan->local_p[slot ^ 1]; X.zero0_n = tp + tu;
    X.zero1 = plan->local_q[slot ^ 1]; X.zero1_n = tq + tz;
    if (plan->total_unc) {
      X.seg_mode = 2; X.nsegs = plan->nsegs; X.segs = plan->segs; X.seg_total = plan->total_unc;
      X.bucket = plan->work; X.dense_err = seg_err; X.peer_staging = plan->peer_stage[slot]; X.seg_scale = inv_ws;
    }
    RUN(conef_orthogonalize_fused(plan->mats, (const int2*)plan->orth_p.tiles, plan->orth_p.n, 0, plan->pu,
                                  plan->eps, plan->peer_p[slot], plan->my_flags, ws, ep1, plan->status, spin,
                                  plan->ppk, plan->np_cols, plan->gram, eb, &X, s));
    plan->launched += conef_orth_last_launches() - 1;
    if (plan->qset_all.simt.n)
      RUN(conef_psgd_q(plan->mats, (const int2*)plan->qset_all.simt.tiles, plan->qset_all.simt.n, plan->work, aux,
                       plan->pu, q_target, plan->max_rank, s));
    const uint32_t ep2 = ebase + (uint32_t)(++*ncoll);
    RUN(conef_psgd_tc_signal(1, plan->mats, plan->tc_maps, plan->qset_all.tc.tiles, plan->qset_all.tc.n, plan->ppk,
                             q_target, plan->max_rank, plan->status, plan->done_word, pflags, ws, plan->rank, ep2,
                             eb, s));
  }

  if (phases & CONEF_PHASE_D) {
    const uint32_t ep2 = ebase + (uint32_t)*ncoll;      // the epoch the Q pass published
    if (peers && plan->wait_kernel)
      RUN(conef_wait_flags_ex(plan->my_flags, ws, ep2, plan->status, spin, eb, s));
    RUN(conef_reduce_q(plan->mats, nm, plan->max_cols, sketch ? plan->tables : nullptr, plan->qz,
                       plan->peer_q[slot], plan->my_flags, ws, ep2, plan->alpha, inv_ws, plan->status, spin, eb, s));
    RUN(conef_psgd_decompress(plan->mats, (const int2*)plan->d_tiles.tiles, plan->d_tiles.n, plan->d_nblk, plan->d_rbu, plan->d_rows,
                              plan->work, plan->pu, plan->qz, 1.0f, plan->sketch, plan->tables, plan->counts,
                              dense_err, plan->alpha, plan->beta, plan->ef_mode, plan->max_rank, plan->d_smem,
                              plan->status, s));
    if (plan->ef_mode == CONEF_EF_SKETCH && plan->d_nblk > 0 && plan->d_nblk < plan->d_tiles.n) ++plan->launched;
    if (plan->topk) {
      RUN(conef_topk_keep(plan->mats, nm, (const int2*)plan->topk_tiles.tiles, plan->topk_tiles.n,
                          plan->dense_err, plan->topk_ratio, plan->topk_scratch, s));
      plan->launched += 6;
    }
  }
  return 0;
}

// eb: null for direct launches (epochs passed by value, continuing from plan->epoch); the device
// epoch word while capturing (epochs relative to it).  *ncoll: collectives enqueued.
static int run_impl(ConefPsgdPlan* plan, int phases, cudaStream_t s, const uint32_t* eb, int* ncoll) {
  plan->launched = 0;
  *ncoll = 0;
  if (plan->fused) return run_fused(plan, phases, s, eb, ncoll);
  const uint32_t ebase = eb ? 0u : plan->epoch;
  const int nm = plan->nm, ws = plan->world, slot = plan->slot & 1;
  const bool symm = plan->has_symm && ws > 1;
  const bool fused_err = plan->ef_mode == CONEF_EF_SKETCH || plan->ef_mode == CONEF_EF_DENSE;
  const float* aux = fused_err ? plan->aux : nullptr;
  const long long tq = plan->total_q, tz = plan->total_z, tp = plan->total_p, tu = plan->total_u;
  float* pmem = plan->pu;          // [0, tp): P
  float* qmem = plan->qz;          // [0, tq): Q
  float* stage = symm ? plan->local_stage[slot] : plan->staging;
  float* p_target = symm ? plan->local_p[slot] : pmem;
  float* dense_err = plan->ef_mode == CONEF_EF_DENSE ? plan->dense_err : nullptr;
  float* seg_err = plan->topk ? nullptr : dense_err;      // error of the uncompressed tensors
  const bool orth_p = !plan->unbiased;
  const float inv_ws = 1.0f / (float)ws;

  if (phases & CONEF_PHASE_P) {
    if (nm) {
      if (plan->fresh) RUN(conef_fill_normal(qmem, tq, plan->seed, s));
      if (!plan->unbiased)
        OK(orth(plan, 1, plan->orth_q, plan->qz, plan->eps, nullptr, nullptr, 1, 0, false, s));
      if (plan->ef_mode == CONEF_EF_SKETCH) {
        // Z = alpha * H^T Q: the sketch records then contribute alpha * unsketch(S) Q to P
        OK(zero_floats(plan->qz + tq, tz, s));
        RUN(conef_sketch_project(plan->mats, nm, plan->max_cols, plan->tables, plan->qz, plan->alpha, 0, s));
      }
    }
    if (plan->total_unc)
      RUN(conef_gather_segments(plan->segs, plan->nsegs, plan->work, seg_err, stage, plan->total_unc, s));
    if (nm) {
      if (plan->p_zero) OK(zero_floats(p_target, tp + tu, s));
      OK(launch_p(plan, aux, p_target, s));
      if (plan->lowrank)      // P += a U (V^T Q)
        OK(correct(plan, plan->corr_p, false, p_target, Term{plan->u_old, plan->qz, plan->qz, plan->alpha},
                   Term{plan->u_old, plan->qz, plan->qz, 0.f}, s));
    }
  }

  if (phases & CONEF_PHASE_Q) {
    if (symm) {
      const uint32_t ep = ebase + (uint32_t)(++*ncoll);
      RUN(conef_signal_peers_ex(plan->peer_flags, ws, plan->rank, ep, eb, s));
      if (nm && orth_p)
        OK(orth(plan, 0, plan->orth_p, plan->pu, plan->eps, plan->peer_p[slot], plan->my_flags, ws,
                ep, true, s, eb));
      else if (nm)
        RUN(conef_allreduce_oneshot_ex(pmem, plan->peer_p[slot], nullptr, plan->my_flags, ws, plan->rank,
                                       ep, tp, inv_ws, plan->status, plan->spin_limit, eb, s));
      else
        RUN(conef_wait_flags_ex(plan->my_flags, ws, ep, plan->status, plan->spin_limit, eb, s));
      if (plan->total_unc)
        RUN(conef_scatter_segments(plan->segs, plan->nsegs, plan->work, plan->peer_stage[slot], ws, nullptr,
                                   inv_ws, seg_err, plan->total_unc, s));
    } else {
      // world > 1 without peer memory: the caller all-reduced staging and P between the phases
      if (plan->total_unc)
        RUN(conef_scatter_segments(plan->segs, plan->nsegs, plan->work, nullptr, 1, stage, inv_ws,
                                   seg_err, plan->total_unc, s));
      if (nm && orth_p)
        OK(orth(plan, 0, plan->orth_p, plan->pu, plan->eps, nullptr, nullptr, 1, 0, true, s));
    }
    if (nm) {
      if (plan->lowrank && symm)      // G V arrived behind the P blocks of the symmetric slot
        OK(copy_floats(plan->pu + tp, p_target + tp, tu, s));
      if (!plan->unbiased) {
        float* q_target = symm ? plan->local_q[slot] : plan->qz;
        if (plan->lowrank) {
          if (plan->q_zero) OK(zero_floats(q_target, tq, s));     // the V blocks behind Q stay
          OK(launch_q(plan, plan->qset_grad, aux, plan->pu, q_target, s));
          OK(correct(plan, plan->corr_q, true, q_target, Term{plan->qz, plan->u_old, plan->pu, plan->alpha},
                     Term{plan->qz, plan->u_old, plan->pu, 0.f}, s));     // Q' += a V (U^T P)
        } else {
          if (plan->q_zero) OK(zero_floats(q_target, tq + tz, s));
          OK(launch_q(plan, plan->qset_all, aux, pmem, q_target, s));
        }
        if (plan->ef_mode == CONEF_EF_SKETCH)     // Q += alpha * H Y with Y = S^T P
          RUN(conef_sketch_project(plan->mats, nm, plan->max_cols, plan->tables, q_target, plan->alpha, 1, s));
      }
    }
  }

  if ((phases & CONEF_PHASE_D) && nm) {
    if (!plan->unbiased && symm) {
      const uint32_t ep = ebase + (uint32_t)(++*ncoll);
      RUN(conef_allreduce_oneshot_ex(qmem, plan->peer_q[slot], plan->peer_flags, plan->my_flags, ws, plan->rank,
                                     ep, tq, inv_ws, plan->status, plan->spin_limit, eb, s));
    }
    if (plan->lowrank) {
      // one power-iteration step of the error factors on T = G + (a+b) U V^T - P Q^T
      const float ab = plan->alpha + plan->beta;
      OK(correct(plan, plan->corr_u, false, plan->pu, Term{plan->u_old, plan->qz, plan->qz, ab},
                 Term{plan->pu, plan->qz, plan->qz, -1.f}, s));           // G V += (a+b) U (V^T V) - P (Q^T V)
      OK(orth(plan, 0, plan->orth_u, plan->pu, 1e-12f, nullptr, nullptr, 1, 0, true, s));
      OK(zero_floats(plan->qz2, tq + tz, s));
      OK(launch_q(plan, plan->qset_err, nullptr, plan->pu, plan->qz2, s));     // G^T U'
      OK(correct(plan, plan->corr_v, true, plan->qz2, Term{plan->qz, plan->u_old, plan->pu, ab},
                 Term{plan->qz, plan->pu, plan->pu, -1.f}, s));           // += (a+b) V (U^T U') - Q (P^T U')
      OK(copy_floats(plan->u_old, plan->pu + tp, tu, s));
      OK(copy_floats(plan->qz + tq, plan->qz2 + tq, tz, s));
    }
    RUN(conef_psgd_decompress(plan->mats, (const int2*)plan->d_tiles.tiles, plan->d_tiles.n, plan->d_nblk, plan->d_rbu, plan->d_rows,
                              plan->work, pmem, qmem, 1.0f, plan->sketch, plan->tables, plan->counts,
                              dense_err, plan->alpha, plan->beta, plan->ef_mode, plan->max_rank,
                              plan->d_smem, plan->status, s));
    if (plan->ef_mode == CONEF_EF_SKETCH && plan->d_nblk > 0 && plan->d_nblk < plan->d_tiles.n) ++plan->launched;
    if (plan->topk) {
      RUN(conef_topk_keep(plan->mats, nm, (const int2*)plan->topk_tiles.tiles, plan->topk_tiles.n,
                          plan->dense_err, plan->topk_ratio, plan->topk_scratch, s));
      plan->launched += 6;
    }
  }
  return 0;
}

extern "C" int conef_psgd_run(ConefPsgdPlan* plan, int phases, cudaStream_t s) {
  int ncoll = 0;
  const int rc = run_impl(plan, phases, s, nullptr, &ncoll);
  plan->epoch += (uint32_t)ncoll;
  return rc;
}

extern "C" int conef_psgd_plan_release(ConefPsgdPlan* plan) {
  for (int i = 0; i < 2; ++i) {
    if (plan->graph_exec[i]) cudaGraphExecDestroy((cudaGraphExec_t)plan->graph_exec[i]);
    plan->graph_exec[i] = nullptr;
    plan->graph_runs[i] = 0;
  }
  return 0;
}

extern "C" int conef_psgd_step(ConefPsgdPlan* plan, cudaStream_t s) {
  const int slot = plan->slot & 1;
  const bool peer = plan->world > 1;
  if (!plan->use_graph || plan->fresh || (peer && (!plan->has_symm || !plan->epoch_word)))
    return conef_psgd_run(plan, CONEF_PHASE_ALL, s);
  if (plan->key_work != plan->work || plan->key_alpha != plan->alpha || plan->key_beta != plan->beta ||
      plan->key_eps != plan->eps) {
    conef_psgd_plan_release(plan);
    plan->key_work = plan->work;
    plan->key_alpha = plan->alpha; plan->key_beta = plan->beta; plan->key_eps = plan->eps;
  }
  if (!plan->graph_exec[slot]) {
    // two direct runs first: every kernel has then set its attributes and loaded its module
    if (plan->graph_runs[slot] < 2) {
      ++plan->graph_runs[slot];
      return conef_psgd_run(plan, CONEF_PHASE_ALL, s);
    }
    cudaGraph_t graph = nullptr;
    int ncoll = 0, rc = 0;
    if (cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
      cudaGetLastError();
      plan->use_graph = 0;
      return conef_psgd_run(plan, CONEF_PHASE_ALL, s);
    }
    rc = run_impl(plan, CONEF_PHASE_ALL, s, peer ? plan->epoch_word : nullptr, &ncoll);
    if (rc == 0 && peer && ncoll) rc = conef_epoch_word(plan->epoch_word, (uint32_t)ncoll, 1, s);
    const cudaError_t ce = cudaStreamEndCapture(s, &graph);
    cudaGraphExec_t exec = nullptr;
    if (rc != 0 || ce != cudaSuccess || graph == nullptr ||
        cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
      if (graph) cudaGraphDestroy(graph);
      cudaGetLastError();
      plan->use_graph = 0;       // nothing was enqueued by the failed capture: run the step directly
      return conef_psgd_run(plan, CONEF_PHASE_ALL, s);
    }
    cudaGraphDestroy(graph);
    plan->graph_exec[slot] = exec;
    plan->graph_launched[slot] = plan->launched + (peer && ncoll ? 1 : 0);
    plan->graph_ncoll[slot] = ncoll;
  }
  if (peer && plan->epoch_shadow != plan->epoch) {
    const int rc = conef_epoch_word(plan->epoch_word, plan->epoch, 0, s);
    if (rc != 0) return rc;
    plan->epoch_shadow = plan->epoch;
  }
  CUDA_OK(cudaGraphLaunch((cudaGraphExec_t)plan->graph_exec[slot], s));
  plan->launched = plan->graph_launched[slot];
  plan->epoch += (uint32_t)plan->graph_ncoll[slot];
  if (peer) plan->epoch_shadow += (uint32_t)plan->graph_ncoll[slot];
  ++plan->graph_replays;
  return 0;
}

// ---------------------------------------------------------------------------
// Random-block family: the order of operations of RandBlockEngine.run in parallel/engine.py.
#define RUNB(call)                     \
  do {                                 \
    int rc_ = (call);                  \
    if (rc_ != 0) return rc_;          \
    ++plan->launched;                  \
  } while (0)

extern "C" int conef_randblock_run(ConefRandblockPlan* plan, int phases, cudaStream_t s) {
  plan->launched = 0;
  const int ws = plan->world, slot = plan->slot & 1;
  if (plan->has_slots && (ws == 1 || plan->has_symm)) {
    // two launches: the gather publishes epoch + 1, the reduce + scatter waits for it (and, in two
    // shots, publishes and waits for epoch + 2)
    const bool peers = ws > 1;
    const uint32_t ep = plan->epoch + 1;
    if (phases & 1) {
      RUNB(conef_randblock_gather_ex(
          plan->blks, (const int2*)plan->tiles.tiles, plan->nblks ? plan->tiles.n : 0, plan->nblk_tiles,
          plan->rows_per_cta, plan->work,
          plan->local_blk[slot], plan->unbiased ? 0.0f : 1.0f,
          plan->ef_mode == CONEF_EF_SKETCH ? plan->sketch : nullptr, plan->tables, plan->counts,
          plan->ef_mode == CONEF_EF_DENSE ? plan->dense_err : nullptr, plan->qcodes, plan->qscales, plan->alpha,
          plan->beta, plan->ef_mode, plan->smem, plan->segs, plan->nsegs, plan->total_unc, plan->local_unc[slot],
          plan->done_word, peers ? plan->peer_flags : nullptr, ws, plan->rank, ep, nullptr, s));
    }
    if (phases & 2) {
      const int two = plan->two_shot && peers;
      if (peers)        // one CTA waits for late peers instead of the whole scatter grid
        RUNB(conef_wait_flags(plan->my_flags, ws, ep, plan->status, plan->spin_limit, s));
      RUNB(conef_randblock_reduce_scatter(
          plan->blks, plan->nblks, plan->segs, plan->nsegs, plan->total_unc, plan->total_block, plan->work,
          plan->peer_unc[slot], plan->peer_blk[slot], two ? plan->peer_red[slot] : nullptr,
          two ? plan->local_red[slot] : nullptr, peers ? plan->peer_flags : nullptr, plan->my_flags, ws, plan->rank,
          ep, nullptr, 1.0f / (float)ws, two, plan->done_word, plan->status, plan->spin_limit, s));
      plan->epoch += two ? 2 : 1;
    }
    return 0;
  }
  const bool symm = plan->has_symm && ws > 1;
  float* stage_unc = symm ? plan->local_unc[slot] : plan->staging_unc;
  float* stage_blk = symm ? plan->local_blk[slot] : plan->staging_blk;
  const float inv_ws = 1.0f / (float)ws;
  if (phases & 1) {
    if (plan->total_unc)
      RUNB(conef_gather_segments(plan->segs, plan->nsegs, plan->work, nullptr, stage_unc, plan->total_unc, s));
    if (plan->nblks)
      // gather scale 0 = unbiased estimator: the kernel divides by the selection probability
      RUNB(conef_randblock_gather(plan->blks, (const int2*)plan->tiles.tiles, plan->tiles.n, plan->nblk_tiles,
                                  plan->rows_per_cta, plan->work, stage_blk, plan->unbiased ? 0.0f : 1.0f,
                                  plan->ef_mode == CONEF_EF_SKETCH ? plan->sketch : nullptr, plan->tables,
                                  plan->counts, plan->ef_mode == CONEF_EF_DENSE ? plan->dense_err : nullptr,
                                  plan->qcodes, plan->qscales, plan->alpha, plan->beta, plan->ef_mode, plan->smem, s));
  }
  if (phases & 2) {
    const float* const* peers_unc = nullptr;
    const float* const* peers_blk = nullptr;
    const float *loc_unc = stage_unc, *loc_blk = stage_blk;
    if (symm) {
      plan->epoch += 1;
      RUNB(conef_signal_peers(plan->peer_flags, ws, plan->rank, plan->epoch, s));
      RUNB(conef_wait_flags(plan->my_flags, ws, plan->epoch, plan->status, plan->spin_limit, s));
      peers_unc = plan->peer_unc[slot];
      peers_blk = plan->peer_blk[slot];
      loc_unc = loc_blk = nullptr;
    }
    if (plan->total_unc)
      RUNB(conef_scatter_segments(plan->segs, plan->nsegs, plan->work, peers_unc, ws, loc_unc, inv_ws, nullptr,
                                  plan->total_unc, s));
    if (plan->nblks)
      RUNB(conef_randblock_scatter(plan->blks, plan->nblks, plan->work, peers_blk, ws, loc_blk, inv_ws,
                                   plan->total_block, s));
  }
  return 0;
}

extern "C" int conef_randblock_plan_size(void) { return (int)sizeof(ConefRandblockPlan); }

// Size of the plan structure, so that a binding can verify its mirror of the layout.
extern "C" int conef_psgd_plan_size(void) { return (int)sizeof(ConefPsgdPlan); }
extern "C" int conef_mat_size(void) { return (int)sizeof(ConefMat); }
