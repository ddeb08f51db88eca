// All-gather -> GEMM with a ranking epilogue, for full-vocabulary evaluation over a row-sharded item table.
//
//   for every query row m (the last-position states of ALL ranks) and every item v of THIS rank's shard:
//       s[m, v] = <x_m, e_v>            bf16 operands, fp32 accumulation on tcgen05 / tensor memory
//   count[m] = #{ v in shard : s[m, v] > pos_score[m]  and  global_id(v) != target[m] }
// so that rank(m) = 1 + sum over ranks of count[m]; the [M, V] logits never exist.
//
// One persistent CTA per SM.  Phase 1 (all-gather, fused): once a peer has raised its "activations
// ready" flag, the CTAs copy that peer's rows into a local staging matrix with plain peer loads, each
// CTA a slice, and bump a per-source counter.  Phase 2: each CTA walks over 256-item tiles of the
// shard; the tile's 256 x D rows stay resident in shared memory while all query blocks stream through
// a 4-stage TMA ring (local rows first; the producer waits, bounded, for the counter of a remote
// source before touching its rows).  tcgen05.mma accumulates 128 x 256 scores in one of two tensor
// memory buffers while the epilogue warps compare the other against pos_score and add per-row counts
// in shared memory; counts are flushed with one atomic per row per CTA.
#include "tcgen05.cuh"

namespace recml {
namespace vrank {
using namespace recml::tc;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 320;     // TMA warp, MMA warp, 8 epilogue warps (two per tensor-memory lane quarter)
constexpr int kMaxWorld = 8;
constexpr int kMaxRows = 4096;     // query rows per call (per-CTA count array in shared memory)

struct Params {
  int M, D, V_local, W, me, rows_per_rank;
  int id_mul, id_add;                 // global item id = local_row * id_mul + id_add
  const __nv_bfloat16* peer_x[kMaxWorld];   // each rank's [rows_per_rank, D] activations (peer addresses)
  __nv_bfloat16* stage;               // local [M, D] staging matrix (rank r's rows at r * rows_per_rank)
  const unsigned long long* ready_flags;   // [W] on this rank: peer r published its activations (>= seq)
  SeqRef seq;
  unsigned int* src_done;             // [W] counters: CTAs that finished copying source r (zero on entry)
  const float* pos_score;             // [M]
  const long long* target;            // [M] global item ids
  int* count;                         // [M] output, zero on entry
  int* status;
};

struct Smem {
  static constexpr int kB = 0;                                  // [256 items, D<=256]: D/64 sub-tiles of 32 KB
  static constexpr int kA = 4 * 32768;                          // ring of [128, 64] stages
  static constexpr int kBars = kA + kStages * 16384;
  static constexpr int kCounts = kBars + 256;
  static constexpr int kTotal = kCounts + kMaxRows * 4 + 1024;
};

__global__ void __launch_bounds__(kThreads, 1)
vocab_rank_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_e, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + Smem::kBars;
  // 0..3 a_full, 4..7 a_empty, 8 b_full, 9 b_empty, 10-11 acc_full, 12-13 acc_empty
  auto bar = [&](int i) { return bars + 8u * i; };
  int* counts = reinterpret_cast<int*>(base_ptr + Smem::kCounts);
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_n = p.D / BK;
  const int m_blocks = (p.M + BM - 1) / BM;
  const int n_tiles = (p.V_local + BN - 1) / BN;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < 2 * kStages; ++i) mbar_init(bar(i), 1);
    mbar_init(bar(8), 1); mbar_init(bar(9), 1);
    mbar_init(bar(10), 1); mbar_init(bar(11), 1);
    mbar_init(bar(12), 256); mbar_init(bar(13), 256);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < p.M; i += kThreads) counts[i] = 0;
  if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), 512);

  // ---- phase 1: fused all-gather of the activations (peer loads -> local staging) ----
  {
    const long long vec_per_rank = static_cast<long long>(p.rows_per_rank) * p.D / 8;   // 16-byte vectors
    for (int q = 0; q < p.W; ++q) {
      const int src = (p.me + q) % p.W;    // own rows first
      __shared__ int src_ok;
      if (threadIdx.x == 0)
        src_ok = (src == p.me || p.ready_flags == nullptr ||
                  wait_flag_ge(p.ready_flags + src, seq_of(p.seq), kDefaultWaitNs, p.status, 64 + src)) ? 1 : 0;
      __syncthreads();
      if (src_ok) {
        const uint4* from = reinterpret_cast<const uint4*>(p.peer_x[src]);
        uint4* to = reinterpret_cast<uint4*>(p.stage + static_cast<long long>(src) * p.rows_per_rank * p.D);
        for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < vec_per_rank;
             i += static_cast<long long>(gridDim.x) * kThreads)
          to[i] = __ldcg(from + i);
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) atomicAdd(p.src_done + src, 1u);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      // the staging matrix was written with ordinary stores by many CTAs: wait for every source's copy
      // to be complete, then make those writes visible to the async (TMA) proxy
      bool ok = true;
      for (int src = 0; src < p.W && ok; ++src) {
        const unsigned long long t0 = global_ns();
        while (atomicAdd(p.src_done + src, 0u) < gridDim.x) {
          __nanosleep(128);
          if (global_ns() - t0 > kDefaultWaitNs) { report(p.status, kPeerTimeout, 80 + src); *abortp = 1; ok = false; break; }
        }
      }
      __threadfence();
      asm volatile("fence.proxy.async;" ::: "memory");
      uint32_t it = 0, nt = 0;
      for (int tile = blockIdx.x; tile < n_tiles && ok && !*abortp; tile += gridDim.x, ++nt) {
        if (!mbar_wait(bar(9), (nt & 1) ^ 1, abortp, p.status, 60)) break;      // previous tile's B no longer read
        mbar_expect_tx(bar(8), kb_n * 32768);
        for (int kb = 0; kb < kb_n; ++kb) tma_load_2d(base + Smem::kB + kb * 32768, &map_e, kb * BK, tile * BN, bar(8));
        for (int mb = 0; mb < m_blocks && ok; ++mb)
          for (int kb = 0; kb < kb_n; ++kb, ++it) {
            const int s = it % kStages;
            if (!mbar_wait(bar(4 + s), ((it / kStages) & 1) ^ 1, abortp, p.status, 61)) { ok = false; break; }
            mbar_expect_tx(bar(s), 16384);
            tma_load_2d(base + Smem::kA + s * 16384, &map_x, kb * BK, mb * BM, bar(s));
          }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16(BM, BN, false, false);
      uint32_t it = 0, acc_it = 0, nt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok && !*abortp; tile += gridDim.x, ++nt) {
        if (!mbar_wait(bar(8), nt & 1, abortp, p.status, 62)) break;
        for (int mb = 0; mb < m_blocks && ok; ++mb, ++acc_it) {
          const int acc = acc_it & 1;
          if (!mbar_wait(bar(12 + acc), ((acc_it >> 1) & 1) ^ 1, abortp, p.status, 63)) { ok = false; break; }
          tc_fence_after();
          for (int kb = 0; kb < kb_n; ++kb, ++it) {
            const int s = it % kStages;
            if (!mbar_wait(bar(s), (it / kStages) & 1, abortp, p.status, 64)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              tc_mma_bf16(tmem_base + acc * BN, make_desc(base + Smem::kA + s * 16384 + k * 32, 16, 1024),
                          make_desc(base + Smem::kB + kb * 32768 + k * 32, 16, 1024), idesc, (kb | k) ? 1u : 0u);
            tc_commit(bar(4 + s));
          }
          if (ok) tc_commit(bar(10 + acc));
        }
        if (ok) tc_commit(bar(9));   // all products that read this B tile have been issued and tracked
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;      // the two warps of a lane quarter take alternate 32-column chunks
    const uint32_t lane_off = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t acc_it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int n0 = tile * BN;
      const bool whole = n0 + BN <= p.V_local;        // no item of the tile lies beyond the shard
      for (int mb = 0; mb < m_blocks; ++mb, ++acc_it) {
        const int acc = acc_it & 1;
        int okw = 1;
        if (lane == 0) okw = mbar_wait(bar(10 + acc), (acc_it >> 1) & 1, abortp, p.status, 65) ? 1 : 0;
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) { ok = false; break; }
        tc_fence_after();
        const int row = mb * BM + quarter * 32 + lane;
        const bool row_ok = row < p.M;
        const float pos = row_ok ? p.pos_score[row] : INFINITY;     // rows past M count nothing
        // local column of this row's own target (it does not compete with itself), -1 when another rank holds it
        int tgt_col = -1;
        if (row_ok) {
          const long long d = p.target[row] - p.id_add;
          if (d >= 0 && d % p.id_mul == 0 && d / p.id_mul < p.V_local) tgt_col = static_cast<int>(d / p.id_mul);
        }
        int c = 0;
#pragma unroll 1
        for (int ch = half; ch < BN / 32; ch += 2) {
          uint32_t v[32];
          tmem_ld32(tmem_base + acc * BN + lane_off + ch * 32, v);
          const int col0 = n0 + ch * 32;
          const bool plain = whole && static_cast<unsigned>(tgt_col - col0) >= 32u;
          if (__all_sync(0xffffffffu, plain)) {
#pragma unroll
            for (int e = 0; e < 32; ++e) c += __uint_as_float(v[e]) > pos ? 1 : 0;
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int item = col0 + e;
              c += (__uint_as_float(v[e]) > pos && item < p.V_local && item != tgt_col) ? 1 : 0;
            }
          }
        }
        tc_fence_before();
        mbar_arrive(bar(12 + acc));
        if (row_ok && c) atomicAdd(counts + row, c);
      }
    }
  }
  if (*abortp) {
    for (int i = 0; i < 64; ++i) __nanosleep(100000);
  }
  tc_fence_before();
  __syncthreads();
  for (int i = threadIdx.x; i < p.M; i += kThreads)
    if (counts[i]) atomicAdd(p.count + i, counts[i]);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace vrank
}  // namespace recml

using namespace recml::vrank;

extern "C" int recml_vocab_rank_struct_size() { return static_cast<int>(sizeof(Params)); }

// item_shard: [V_local, D] bf16 (row-major); D in {64, 128, 192, 256}; M <= 4096 and a multiple of W.
extern "C" int recml_vocab_rank(const void* item_shard, const Params* p, cudaStream_t stream) {
  if (p->M <= 0 || p->V_local <= 0) return 0;
  if (p->M > kMaxRows || p->D % 64 || p->D > 256 || p->W > kMaxWorld) return -10;
  CUtensorMap mx, me;
  if (recml::tc::make_map_bf16(&mx, p->stage, p->M, p->D, p->D, BM) ||
      recml::tc::make_map_bf16(&me, item_shard, p->V_local, p->D, p->D, BN))
    return -2;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(vocab_rank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal) != cudaSuccess)
      return -3;
    configured = true;
  }
  const int n_tiles = (p->V_local + BN - 1) / BN;
  const int grid = n_tiles < recml::tc::sm_count() ? n_tiles : recml::tc::sm_count();
  // every CTA takes part in the copy phase and later waits for all of them: the grid must be co-resident,
  // which one CTA per SM (launch bounds, ~213 KB of shared memory) guarantees for grid <= #SMs
  vocab_rank_kernel<<<grid, kThreads, Smem::kTotal, stream>>>(mx, me, *p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

namespace recml {
namespace vrank {
__global__ void publish_kernel(unsigned long long* const* flags, int W, SeqRef seq) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();
    const unsigned long long v = seq_of(seq);
    for (int r = 0; r < W; ++r)
      if (flags[r] != nullptr) st_release_sys(flags[r], v);
  }
}
}  // namespace vrank
}  // namespace recml

struct PublishArgs { unsigned long long* flags[recml::vrank::kMaxWorld]; };

__global__ void publish_kernel_byval(PublishArgs a, int W, recml::SeqRef seq) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();
    const unsigned long long v = recml::seq_of(seq);
    for (int r = 0; r < W; ++r)
      if (a.flags[r] != nullptr) recml::st_release_sys(a.flags[r], v);
  }
}

// Raises flag = seq on every rank (stream-ordered after whatever produced the published data).
extern "C" int recml_publish_flags(const PublishArgs* args, int W, const recml::SeqRef* seq, cudaStream_t stream) {
  publish_kernel_byval<<<1, 32, 0, stream>>>(*args, W, *seq);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
