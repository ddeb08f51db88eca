// bf16 GEMM on 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   D[M,N] = epilogue( A[M,K] · B[N,K]^T )      fp32 accumulation in tensor memory
//
// One persistent CTA per SM walks over 128 x BN output tiles.  Warp roles:
//   warp 0      TMA producer: cp.async.bulk.tensor (2-D tiled, 128-byte swizzle, no cluster
//               broadcast) fills a ring of shared-memory stages and signals "full" mbarriers
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN, K=16) and
//               releases stages / publishes accumulators with tcgen05.commit
//   warps 2..9  epilogue: tcgen05.ld the accumulator (two warps per 32-lane quarter, taking
//               alternate 64-column slabs), apply the fused epilogue, store bf16 / fp32 rows
// Two accumulator buffers (2 x BN columns of tensor memory) let the epilogue of tile i
// overlap the main loop of tile i+1.
//
// Operand layouts.  Each operand is given as a row-major matrix in global memory together
// with a flag saying which of its two dims is contiguous:
//   "K-major"  A stored [M,K] / B stored [N,K]   (contraction dim contiguous)
//   "MN-major" A stored [K,M] / B stored [K,N]   (output dim contiguous)
// so that Y = X·W^T (both K-major), dX = dY·W (B MN-major) and dW = dY^T·X (both MN-major)
// all run without materialising a transpose.
//
// Every wait is bounded (see common.cuh); on expiry the CTA drains and frees its tensor
// memory before returning, and the launcher's status word is set.
#include <cstdlib>

#include "tcgen05.cuh"

namespace recml {
namespace gemm {
using namespace recml::tc;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kThreads = 320;   // TMA warp, MMA warp, 8 epilogue warps

enum Epilogue : int {
  kEpiLinear = 0,    // D = act(acc + bias)
  kEpiCross = 1,     // V = acc + bias (optional store to out2); D = aux0 * V + aux1
  kEpiMaskRelu = 2,  // D = acc * (aux0 > 0)              (ReLU backward fused in dgrad)
  kEpiMulAdd = 3,    // D = acc * aux0 (+ aux1)           (DCN input-gradient paths)
  kEpiAdd = 4,       // D = acc + aux0 (+ aux1)           (residual / skip gradients)
};

struct Params {
  int M, N, K;
  void* d;            // bf16 or fp32 [M, ldd]
  int ldd;
  int out_f32;        // 1: D is fp32
  int accumulate;     // 1: D += result (fp32 output only)
  int split_k;        // >1: the K loop is cut into split_k ranges handled by different CTAs; partial
                      //     results are added to the fp32 output with atomics (output pre-zeroed)
  const float* bias;  // [N] or null
  int relu;
  int epi;
  const __nv_bfloat16* aux0;  // [M, ldaux]
  const __nv_bfloat16* aux1;  // [M, ldaux]
  int ldaux;
  __nv_bfloat16* out2;        // optional second output [M, ldd] (kEpiCross: V)
  int* status;
};

template <int BN>
struct Cfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStages = (BN == 256) ? 3 : 4;
  // per epilogue warp: one staging set of two 4 KB [32 rows, 64 cols] bf16 boxes (auxiliary operands come in,
  // results are written over them and go out)
  static constexpr int kEpi = 4 * 4 * 4096;
  static constexpr int kSmem = kStages * (kStageA + kStageB) + kEpi + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int kTmemCols = 2 * BN;
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_d2,
            const __grid_constant__ CUtensorMap map_x0, const __grid_constant__ CUtensorMap map_x1,
            const Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = base;
  const uint32_t smem_b = base + C::kStages * C::kStageA;
  const uint32_t epi_smem = smem_b + C::kStages * C::kStageB;
  uint8_t* epi_ptr = smem_raw + (epi_smem - smem_u32(smem_raw));
  const uint32_t bars = epi_smem + C::kEpi;
  // barrier slots (8 bytes each): full[S], empty[S], tmem_full[2], tmem_empty[2], aux_full[4 warps]
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  auto tfull_bar = [&](int s) { return bars + 8u * (2 * C::kStages + s); };
  auto tempty_bar = [&](int s) { return bars + 8u * (2 * C::kStages + 2 + s); };
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int split_k = p.split_k > 1 ? p.split_k : 1;
  const int num_tiles = m_tiles * n_tiles * split_k;   // work units
  const int k_blocks_total = (p.K + BK - 1) / BK;
  const int kb_per = (k_blocks_total + split_k - 1) / split_k;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 256);
    }
    for (int w = 0; w < 8; ++w) mbar_init(bars + 8u * (2 * C::kStages + 4 + w), 1);   // 4 epilogue warps x 2 staging sets
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_base_slot), C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abortp; tile += gridDim.x) {
        const int tl = tile / split_k, ks = tile % split_k;
        const int m0 = (tl / n_tiles) * BM, n0 = (tl % n_tiles) * BN;
        const int kb0 = ks * kb_per, kb1 = min(k_blocks_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % C::kStages;
          if (!mbar_wait(empty_bar(s), ((it / C::kStages) & 1) ^ 1, abortp, p.status, 10)) break;
          mbar_expect_tx(full_bar(s), C::kStageA + C::kStageB);
          const uint32_t sa = smem_a + s * C::kStageA, sb = smem_b + s * C::kStageB;
          const int k0 = kb * BK;
          if (A_MN) {
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &map_a, m0 + 64 * j, k0, full_bar(s));
          } else {
            tma_load_2d(sa, &map_a, k0, m0, full_bar(s));
          }
          if (B_MN) {
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &map_b, n0 + 64 * j, k0, full_bar(s));
          } else {
            tma_load_2d(sb, &map_b, k0, n0, full_bar(s));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      // instruction descriptor: D=f32, A=B=bf16, majors, N>>3, M>>4
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) |
                             ((B_MN ? 1u : 0u) << 16) | (static_cast<uint32_t>(BN >> 3) << 17) |
                             (static_cast<uint32_t>(BM >> 4) << 24);
      // K-major: rows of 128 B, 8-row groups 1024 B apart; advance 32 B per K=16.
      // MN-major: 64-element atoms, 8-k groups 1024 B apart, next 64-wide atom 8192 B on;
      //           advance 2048 B per K=16.
      const uint32_t a_lbo = A_MN ? 8192u : 16u, b_lbo = B_MN ? 8192u : 16u;
      const uint32_t a_step = A_MN ? 2048u : 32u, b_step = B_MN ? 2048u : 32u;
      uint32_t it = 0, t = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abortp; tile += gridDim.x, ++t) {
        const int acc = t & 1;
        if (!mbar_wait(tempty_bar(acc), ((t >> 1) & 1) ^ 1, abortp, p.status, 20)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        bool ok = true;
        const int ks = tile % split_k;
        const int kb0 = ks * kb_per, kb1 = min(k_blocks_total, kb0 + kb_per);
        if (kb0 >= kb1) {           // empty K range (cannot happen for kb_per >= 1 splits that exist)
          tc_commit(tfull_bar(acc));
          continue;
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % C::kStages;
          if (!mbar_wait(full_bar(s), (it / C::kStages) & 1, abortp, p.status, 21)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_a + s * C::kStageA, sb = smem_b + s * C::kStageB;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_desc(sa + k * a_step, a_lbo, 1024);
            const uint64_t bdesc = make_desc(sb + k * b_step, b_lbo, 1024);
            tc_mma_bf16(tmem_d, adesc, bdesc, idesc, ((kb - kb0) | k) ? 1u : 0u);
          }
          tc_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));  // accumulator complete
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    // bf16 outputs: the two warps of a lane quarter own the same 32 rows of the tile and take alternate
    // 64-column slabs.  Per slab a warp (1) TMA-loads the 32 x 64 boxes of the auxiliary operands into
    // its private staging set, (2) reads the accumulator from tensor memory, applies the epilogue and
    // writes the bf16 results OVER the auxiliary boxes (same thread, same 16-byte chunk), (3) hands the
    // boxes to TMA stores.  While one warp waits for its loads or for its store to drain, its sibling
    // computes, so the quarter keeps a slab in flight at every stage.  All global traffic of the
    // epilogue is full 128-byte lines and only __syncwarp is needed.  fp32 outputs (weight gradients)
    // are written directly: a thread's 32 floats already are one full line.
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32)
    const int sub = (warp - 2) >> 2;         // which of the quarter's two warps
    const uint32_t my_smem = epi_smem + quarter * 16384 + sub * 8192;
    uint8_t* st = epi_ptr + quarter * 16384 + sub * 8192;
    const uint32_t aux_bar = bars + 8u * (2 * C::kStages + 4 + quarter * 2 + sub);
    const int n_aux = p.epi == kEpiLinear ? 0 : ((p.epi == kEpiCross || ((p.epi == kEpiMulAdd || p.epi == kEpiAdd) && p.aux1 != nullptr)) ? 2 : 1);
    const bool cross = p.epi == kEpiCross;
    auto slabs_of = [&](int tl) {
      const int rem = p.N - (tl % n_tiles) * BN;
      return rem >= BN ? BN / 64 : (rem + 63) / 64;
    };
    uint32_t aux_uses = 0;      // completed phases of this warp's aux barrier
    uint32_t t = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++t) {
      const int tl = tile / split_k;
      const int m0 = (tl / n_tiles) * BM, n0 = (tl % n_tiles) * BN;
      const int acc = t & 1;
      {
        int okw = 1;
        if (lane == 0) okw = mbar_wait(tfull_bar(acc), (t >> 1) & 1, abortp, p.status, 30) ? 1 : 0;
        if (!__shfl_sync(0xffffffffu, okw, 0)) break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (!p.out_f32) {
        const int row0 = m0 + quarter * 32;
        bool ok = true;
        const int n_slabs = slabs_of(tl);
#pragma unroll 1
        for (int sl = sub; sl < n_slabs && ok; sl += 2) {
          const int col0 = n0 + sl * 64;
          if (lane == 0) {
            // this warp's previous store has finished reading the staging set
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            if (n_aux > 0) {
              mbar_expect_tx(aux_bar, 4096u * n_aux);
              tma_load_2d(my_smem, &map_x0, col0, row0, aux_bar);
              if (n_aux == 2) tma_load_2d(my_smem + 4096, &map_x1, col0, row0, aux_bar);
            }
          }
          __syncwarp();
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t r[32];
            tmem_ld32(taddr + sl * 64 + hh * 32, r);
            if (hh == 0 && n_aux > 0) {
              int okw = 1;
              if (lane == 0) okw = mbar_wait(aux_bar, aux_uses & 1u, abortp, p.status, 31) ? 1 : 0;
              ++aux_uses;
              if (!__shfl_sync(0xffffffffu, okw, 0)) { ok = false; break; }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = col0 + hh * 32 + g * 8;
              const int chunk = ((hh * 4 + g) ^ (lane & 7)) * 16 + lane * 128;
              float x[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(r[g * 8 + j]);
              if (p.bias != nullptr && col < p.N) {
                const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + col));
                const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + col + 4));
                x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w;
                x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
              }
              int out_off = 0;      // where the result goes inside the set: over aux0, or over aux1 for the cross epilogue
              if (p.epi == kEpiLinear) {
                if (p.relu) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) x[j] = fmaxf(x[j], 0.f);
                }
              } else {
                const uint4 a0 = *reinterpret_cast<const uint4*>(st + chunk);
                const uint32_t a0w[4] = {a0.x, a0.y, a0.z, a0.w};
                if (cross) {
                  const uint4 a1 = *reinterpret_cast<const uint4*>(st + 4096 + chunk);
                  const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w};
                  // second output V = acc + bias replaces the x0 chunk this thread has just read
                  *reinterpret_cast<uint4*>(st + chunk) =
                      make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    x[2 * j] = bf16_lo(a0w[j]) * x[2 * j] + bf16_lo(a1w[j]);
                    x[2 * j + 1] = bf16_hi(a0w[j]) * x[2 * j + 1] + bf16_hi(a1w[j]);
                  }
                  out_off = 4096;
                } else if (p.epi == kEpiMaskRelu) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    x[2 * j] = bf16_lo(a0w[j]) > 0.f ? x[2 * j] : 0.f;
                    x[2 * j + 1] = bf16_hi(a0w[j]) > 0.f ? x[2 * j + 1] : 0.f;
                  }
                } else if (p.epi == kEpiAdd) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    x[2 * j] += bf16_lo(a0w[j]);
                    x[2 * j + 1] += bf16_hi(a0w[j]);
                  }
                  if (n_aux == 2) {
                    const uint4 a1 = *reinterpret_cast<const uint4*>(st + 4096 + chunk);
                    const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      x[2 * j] += bf16_lo(a1w[j]);
                      x[2 * j + 1] += bf16_hi(a1w[j]);
                    }
                  }
                } else {  // kEpiMulAdd
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    x[2 * j] *= bf16_lo(a0w[j]);
                    x[2 * j + 1] *= bf16_hi(a0w[j]);
                  }
                  if (n_aux == 2) {
                    const uint4 a1 = *reinterpret_cast<const uint4*>(st + 4096 + chunk);
                    const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      x[2 * j] += bf16_lo(a1w[j]);
                      x[2 * j + 1] += bf16_hi(a1w[j]);
                    }
                  }
                }
              }
              *reinterpret_cast<uint4*>(st + out_off + chunk) =
                  make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
            }
          }
          if (!ok) break;
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&map_d, col0, row0, my_smem + (cross ? 4096u : 0u));
            if (cross && p.out2 != nullptr) tma_store_2d(&map_d2, col0, row0, my_smem);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        if (!ok) break;
      } else {
#pragma unroll 1
        for (int c = sub; c < BN / 32; c += 2) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;  // warp-uniform
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          if (!row_ok) continue;
          const size_t off = static_cast<size_t>(row) * p.ldd + col0;
          const size_t aoff = static_cast<size_t>(row) * p.ldaux + col0;
  #pragma unroll
          for (int v = 0; v < 4; ++v) {  // 4 groups of 8 columns
            if (col0 + v * 8 >= p.N) break;
            float x[8];
  #pragma unroll
            for (int j = 0; j < 8; ++j) x[j] = __uint_as_float(r[v * 8 + j]);
            if (p.bias != nullptr) {
              const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + v * 8));
              const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + v * 8 + 4));
              x[0] += b0.x; x[1] += b0.y; x[2] += b0.z; x[3] += b0.w;
              x[4] += b1.x; x[5] += b1.y; x[6] += b1.z; x[7] += b1.w;
            }
            if (p.epi == kEpiLinear) {
              if (p.relu) {
  #pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = fmaxf(x[j], 0.f);
              }
            } else {
              const uint4 a0 = __ldg(reinterpret_cast<const uint4*>(p.aux0 + aoff + v * 8));
              const uint32_t a0w[4] = {a0.x, a0.y, a0.z, a0.w};
              if (p.epi == kEpiCross) {
                if (p.out2 != nullptr) {
                  uint4 o;
                  o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]);
                  o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
                  *reinterpret_cast<uint4*>(p.out2 + off + v * 8) = o;
                }
                const uint4 a1 = __ldg(reinterpret_cast<const uint4*>(p.aux1 + aoff + v * 8));
                const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w};
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  x[2 * j] = bf16_lo(a0w[j]) * x[2 * j] + bf16_lo(a1w[j]);
                  x[2 * j + 1] = bf16_hi(a0w[j]) * x[2 * j + 1] + bf16_hi(a1w[j]);
                }
              } else if (p.epi == kEpiMaskRelu) {
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  x[2 * j] = bf16_lo(a0w[j]) > 0.f ? x[2 * j] : 0.f;
                  x[2 * j + 1] = bf16_hi(a0w[j]) > 0.f ? x[2 * j + 1] : 0.f;
                }
              } else if (p.epi == kEpiAdd) {
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  x[2 * j] += bf16_lo(a0w[j]);
                  x[2 * j + 1] += bf16_hi(a0w[j]);
                }
                if (p.aux1 != nullptr) {
                  const uint4 a1 = __ldg(reinterpret_cast<const uint4*>(p.aux1 + aoff + v * 8));
                  const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w};
  #pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    x[2 * j] += bf16_lo(a1w[j]);
                    x[2 * j + 1] += bf16_hi(a1w[j]);
                  }
                }
              } else {  // kEpiMulAdd
  #pragma unroll
                for (int j = 0; j < 4; ++j) {
                  x[2 * j] *= bf16_lo(a0w[j]);
                  x[2 * j + 1] *= bf16_hi(a0w[j]);
                }
                if (p.aux1 != nullptr) {
                  const uint4 a1 = __ldg(reinterpret_cast<const uint4*>(p.aux1 + aoff + v * 8));
                  const uint32_t a1w[4] = {a1.x, a1.y, a1.z, a1.w};
  #pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    x[2 * j] += bf16_lo(a1w[j]);
                    x[2 * j + 1] += bf16_hi(a1w[j]);
                  }
                }
              }
            }
            if (p.out_f32) {
              float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.d) + off + v * 8);
              float4 o0 = make_float4(x[0], x[1], x[2], x[3]), o1 = make_float4(x[4], x[5], x[6], x[7]);
              if (split_k > 1) {
                atomicAdd(dst, o0);
                atomicAdd(dst + 1, o1);
                continue;
              }
              if (p.accumulate) {
                const float4 c0 = dst[0], c1 = dst[1];
                o0.x += c0.x; o0.y += c0.y; o0.z += c0.z; o0.w += c0.w;
                o1.x += c1.x; o1.y += c1.y; o1.z += c1.z; o1.w += c1.w;
              }
              dst[0] = o0; dst[1] = o1;
            } else {
              uint4 o;
              o.x = pack_bf16(x[0], x[1]); o.y = pack_bf16(x[2], x[3]);
              o.z = pack_bf16(x[4], x[5]); o.w = pack_bf16(x[6], x[7]);
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.d) + off + v * 8) = o;
            }
          }
        }
  
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // ------------------------------ teardown ------------------------------
  if (*abortp) {
    // give copies / MMAs already in flight time to land before shared and tensor memory go away
    for (int i = 0; i < 64; ++i) __nanosleep(100000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---- host side ---------------------------------------------------------------------------------
static int make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows) {
  return make_map_bf16(map, ptr, rows, cols, ld, box_rows);
}

template <int BN, bool A_MN, bool B_MN>
static int launch(const void* a, int lda, const void* b, int ldb, const Params& p, cudaStream_t stream) {
  CUtensorMap ma, mb;
  int rc;
  // K-major operand: matrix [MN, K], box [BM|BN rows, 64 k]; MN-major: matrix [K, MN], box [64 k rows, 64 mn]
  rc = A_MN ? make_map(&ma, a, p.K, p.M, lda, 64) : make_map(&ma, a, p.M, p.K, lda, BM);
  if (rc) return rc;
  rc = B_MN ? make_map(&mb, b, p.K, p.N, ldb, 64) : make_map(&mb, b, p.N, p.K, ldb, BN);
  if (rc) return rc;
  // bf16 outputs / auxiliary operands move through [32 rows, 64 cols] boxes (one per epilogue warp)
  CUtensorMap md, md2, mx0, mx1;
  if (!p.out_f32) {
    if (make_map(&md, p.d, p.M, p.N, p.ldd, 32)) return -5;
  } else {
    md = ma;
  }
  md2 = md; mx0 = md; mx1 = md;
  if (!p.out_f32 && p.out2 != nullptr && make_map(&md2, p.out2, p.M, p.N, p.ldd, 32)) return -5;
  if (!p.out_f32 && p.aux0 != nullptr && make_map(&mx0, p.aux0, p.M, p.N, p.ldaux, 32)) return -5;
  if (!p.out_f32 && p.aux1 != nullptr && make_map(&mx1, p.aux1, p.M, p.N, p.ldaux, 32)) return -5;
  auto kern = gemm_kernel<BN, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmem) != cudaSuccess)
      return -3;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * (p.split_k > 1 ? p.split_k : 1);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kThreads, Cfg<BN>::kSmem, stream>>>(ma, mb, md, md2, mx0, mx1, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace gemm
}  // namespace recml

// D[M,N] = epi(A·B^T).  a_mn / b_mn: 0 = operand stored [rows, K] (K contiguous), 1 = stored [K, rows].
// Leading dims are in elements and must be multiples of 8 (16-byte TMA strides); N must be a multiple of 8.
// Returns 0 on a successful launch, negative on bad arguments / set-up failure.
extern "C" int recml_gemm_bf16(const void* a, int lda, int a_mn, const void* b, int ldb, int b_mn, void* d,
                               int ldd, int out_f32, int accumulate, int M, int N, int K, const float* bias,
                               int relu, int epi, const void* aux0, const void* aux1, int ldaux, void* out2,
                               int split_k, int* status, cudaStream_t stream) {
  using namespace recml::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (ldd % 4) || (!out_f32 && (ldd % 8))) return -10;
  if (epi != kEpiLinear && (aux0 == nullptr || (ldaux % 8))) return -11;
  if (epi != kEpiLinear && out_f32) return -14;   // fused epilogues produce bf16
  if ((reinterpret_cast<uintptr_t>(aux0) | reinterpret_cast<uintptr_t>(aux1) | reinterpret_cast<uintptr_t>(out2)) & 15) return -12;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(d)) & 15) return -12;
  Params p;
  p.M = M; p.N = N; p.K = K; p.d = d; p.ldd = ldd; p.out_f32 = out_f32; p.accumulate = accumulate;
  p.bias = bias; p.relu = relu; p.epi = epi;
  p.aux0 = static_cast<const __nv_bfloat16*>(aux0); p.aux1 = static_cast<const __nv_bfloat16*>(aux1);
  p.ldaux = ldaux; p.out2 = static_cast<__nv_bfloat16*>(out2); p.status = status;
  {
    const int kb = (K + BK - 1) / BK;
    if (split_k > kb) split_k = kb;
    if (split_k > 1 && (!out_f32 || epi != kEpiLinear || bias != nullptr || relu)) return -13;
    // every split must own at least one k-block
    while (split_k > 1 && ((kb + split_k - 1) / split_k) * (split_k - 1) >= kb) --split_k;
    p.split_k = split_k > 1 ? split_k : 1;
  }
  // Tile width: 256 columns amortise the operand traffic of long-K products; products whose epilogue streams
  // auxiliary operands through the tile (cross / add / mask epilogues) are bound by that epilogue when K is
  // short, and then twice as many half-width tiles keep more of it in flight and balance the last wave.
  static const int forced_bn = [] { const char* e = getenv("RECML_GEMM_BN"); return e ? atoi(e) : 0; }();
  bool wide = N > 128;
  if (wide && epi != kEpiLinear && !out_f32 && K <= 1024 &&
      static_cast<long long>((M + BM - 1) / BM) * ((N + 255) / 256) < 8LL * sm_count()) wide = false;
  if (forced_bn == 128) wide = false;
  if (forced_bn == 256) wide = N > 128;
  if (!a_mn && !b_mn) return wide ? launch<256, false, false>(a, lda, b, ldb, p, stream)
                                  : launch<128, false, false>(a, lda, b, ldb, p, stream);
  if (!a_mn && b_mn) return wide ? launch<256, false, true>(a, lda, b, ldb, p, stream)
                                 : launch<128, false, true>(a, lda, b, ldb, p, stream);
  if (a_mn && b_mn) return wide ? launch<256, true, true>(a, lda, b, ldb, p, stream)
                                : launch<128, true, true>(a, lda, b, ldb, p, stream);
  return wide ? launch<256, true, false>(a, lda, b, ldb, p, stream)
              : launch<128, true, false>(a, lda, b, ldb, p, stream);
}
