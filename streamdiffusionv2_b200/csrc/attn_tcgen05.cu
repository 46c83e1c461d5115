// Attention of new queries over the K/V cache on the sm_100a tensor cores.
//
// One CTA per (pair of 128-row query tiles, head, cache row).  Warp roles:
//   warp 0      TMA producer: Q tiles once, then K_0 and the pairs (V_j, K_{j+1}) through a ring of 32 KB slots;
//               a pair is what one key-tile step consumes, so it has one "landed" and one "released" barrier
//   warp 1      MMA issuer (one thread): S = Q K^T and O += P V with tcgen05.mma, fp32 in TMEM
//   warps 4-7   softmax for query tile 0 (one thread per query row = one TMEM lane)
//   warps 8-11  softmax for query tile 1
// The two query tiles share every K/V tile and alternate on the tensor pipe, so one tile's
// softmax overlaps the other tile's MMAs.  P (bf16) is written back into the TMEM columns of S
// and consumed as the A operand of the P V product; V is consumed MN-major straight from the
// [kv, d] tile the TMA delivered.  O is rescaled lazily: only when a row maximum grows by more
// than 2^8 is the accumulator in TMEM touched, by the softmax warps themselves.
//
// TMEM columns (512): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_i aliases S_i[0,64).
// Shared memory: Q0 Q1 (32 KB each) | kSlots x 32 KB K/V ring | mbarriers.
// Every tile is two TMA boxes of 64 bf16 x 128 rows with the 128-byte swizzle.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "ptx.cuh"
#include "sdv2_internal.h"

namespace sdv2 {
namespace attn {

constexpr int kBM = 128;   // query rows per tile
constexpr int kBN = 128;   // kv rows per tile
constexpr int kHD = 128;   // head dim
constexpr uint32_t kTileBytes = kBN * kHD * 2;
constexpr uint32_t kHalfTile = kTileBytes / 2;  // one 64-column box
constexpr int kSlots = 5;
constexpr int kThreads = 384;
constexpr uint32_t kSmemQ = 0;
constexpr uint32_t kSmemKV = 2 * kTileBytes;
constexpr uint32_t kSmemBar = kSmemKV + kSlots * kTileBytes;
constexpr uint32_t kSmemBytes = kSmemBar + 256 + 1024;  // + alignment slack

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;

// barrier indices.  K_0 has a barrier of its own; after it the ring carries pairs (V_g, K_{g+1}), the two
// tiles one key-tile step of the issuer consumes and releases together, so that step needs one wait and
// one commit for both.  Three barriers of each kind suffice: the producer is at most two pairs ahead.
constexpr int kPairBars = 3;
constexpr int kBarQFull = 0;                        // [2]
constexpr int kBarK0Full = 2;                       // K_0 landed
constexpr int kBarPairFull = 3;                     // [kPairBars] V_g and K_{g+1} landed
constexpr int kBarPairDone = 3 + kPairBars;         // [kPairBars] every MMA reading V_g or K_{g+1} (or older) completed
constexpr int kBarSFull = 3 + 2 * kPairBars;        // [2]
constexpr int kBarPFull = kBarSFull + 2;            // [2]
constexpr int kBarOFull = kBarPFull + 2;            // [2]
constexpr int kBarPHalf = kBarOFull + 2;            // [2] first 64 key columns of P written
constexpr int kNumBars = kBarPHalf + 2;
static_assert(kNumBars * 8 + 16 <= 256, "barrier block too small");
static_assert(kSlots >= 5, "pair g overwrites the tiles of pairs g-3 and g-2: needs five slots");

constexpr uint32_t kIdescQK = umma_idesc_bf16(kBM, kBN, false, false);
constexpr uint32_t kIdescPV = umma_idesc_bf16(kBM, kHD, false, true);

constexpr float kRescaleThreshold = 8.0f;  // log2 units

// S[stage] = Q[stage] (128 x 128, K-major) * K_tile^T (128 x 128, K-major); 8 steps of K = 16.
__device__ __forceinline__ void issue_qk(uint32_t tmem_s, uint32_t sq, uint32_t sk) {
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t off = (k >> 2) * kHalfTile + (k & 3) * 32;
    umma_ss(tmem_s, umma_smem_desc(sq + off, 16, 1024), umma_smem_desc(sk + off, 16, 1024), kIdescQK,
            k > 0 ? 1u : 0u);
  }
}
// O[stage] (+)= P[stage] (128 x 128 bf16 in TMEM, 8 columns per K step) * V_tile (kv x d, MN-major).
// k_begin..k_end select 16-key steps, so that the first half of a tile can be issued while the
// softmax warps are still producing the second half of P.
// a_from_smem (the rate measurement only): A is the K-major shared-memory tile at sa instead of P.
__device__ __forceinline__ void issue_pv(uint32_t tmem_o, uint32_t tmem_p, uint32_t sv, bool accumulate,
                                         int k_begin = 0, int k_end = 8, bool a_from_smem = false, uint32_t sa = 0) {
#pragma unroll
  for (int k = k_begin; k < k_end; ++k) {
    const uint32_t acc = (accumulate || k > k_begin) ? 1u : 0u;
    const uint64_t b_desc = umma_smem_desc(sv + k * 2048, kHalfTile, 1024);
    if (a_from_smem)
      umma_ss(tmem_o, umma_smem_desc(sa + (k >> 2) * kHalfTile + (k & 3) * 32, 16, 1024), b_desc, kIdescPV, acc);
    else
      umma_ts(tmem_o, tmem_p + k * 8, b_desc, kIdescPV, acc);
  }
}

// kTrace: CTA 0 records cycle stamps of its issuing thread and of one softmax thread per query tile
// (a measurement aid, launched only when SDV2_ATTN_TRACE is set; the normal instantiation has none of it).
template <bool kTrace>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t bar0 = base + kSmemBar;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + kSmemBar + kNumBars * 8);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + kSmemBar + kNumBars * 8 + 4);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;

  // work item: a whole (query tile pair, head, row) tile, or one key range of a tail tile
  int tile = blockIdx.x, part = -1;
  if (tile >= p.n_full) {
    const int r = tile - p.n_full;
    tile = p.n_full + r / p.split;
    part = r - (r / p.split) * p.split;
  }
  const int pt = tile % p.pair_tiles;
  const int hb = tile / p.pair_tiles;
  const int h = hb % p.heads;
  const int b = hb / p.heads;
  const int q0 = pt * (2 * kBM);
  const bool two_tiles = q0 + kBM < p.q_tokens;
  const int seq_len = p.seq_lens[b];
  const int n_kv_all = (seq_len + kBN - 1) / kBN;
  const int j0 = part < 0 ? 0 : static_cast<int>(static_cast<int64_t>(part) * n_kv_all / p.split);
  const int j1 = part < 0 ? n_kv_all : static_cast<int>(static_cast<int64_t>(part + 1) * n_kv_all / p.split);
  const int n_kv = j1 - j0;  // key tiles of this item (the host keeps split <= n_kv_all, so >= 1)
  const int bk = p.kv_row_broadcast ? 0 : b;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) mbar_init(bar(kBarQFull + i), 1);
    mbar_init(bar(kBarK0Full), 1);
    for (int i = 0; i < kPairBars; ++i) {
      mbar_init(bar(kBarPairFull + i), 1);
      mbar_init(bar(kBarPairDone + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(kBarSFull + i), 1);
      mbar_init(bar(kBarPFull + i), kBM);
      mbar_init(bar(kBarPHalf + i), kBM);
      mbar_init(bar(kBarOFull + i), 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  auto stamp = [&](int j, int k) {
    if (kTrace && blockIdx.x == 0 && p.trace != nullptr && j < 256) p.trace[j * 32 + k] = clock64();
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int n_q = two_tiles ? 2 : 1;
      for (int s = 0; s < n_q; ++s) {
        mbar_expect_tx(bar(kBarQFull + s), kTileBytes);
        tma_load_4d(base + kSmemQ + s * kTileBytes, &tm_q, bar(kBarQFull + s), 0, h, q0 + s * kBM, b);
        tma_load_4d(base + kSmemQ + s * kTileBytes + kHalfTile, &tm_q, bar(kBarQFull + s), 64, h,
                    q0 + s * kBM, b);
      }
      auto slot_addr = [&](int it) { return base + kSmemKV + (it % kSlots) * kTileBytes; };
      auto load_tile = [&](const CUtensorMap* tm, int it, int kv_tile, uint32_t full_bar) {
        tma_load_4d(slot_addr(it), tm, full_bar, 0, h, (j0 + kv_tile) * kBN, bk);
        tma_load_4d(slot_addr(it) + kHalfTile, tm, full_bar, 64, h, (j0 + kv_tile) * kBN, bk);
      };
      mbar_expect_tx(bar(kBarK0Full), kTileBytes);
      load_tile(&tm_k, 0, 0, bar(kBarK0Full));
      bool ok = true;
      int issued = 0;  // pairs requested
      for (int g = 0; g < n_kv && ok; ++g) {  // pair g = items 2g+1 (V_g) and 2g+2 (K_{g+1})
        // the slots of pair g held K_{g-2} and V_{g-2}: free once step g-2 of the issuer has completed
        if (g >= 2)
          ok = mbar_wait(bar(kBarPairDone + (g - 2) % kPairBars), ((g - 2) / kPairBars) & 1, abort_flag, p.status,
                         WAIT_KV_EMPTY);
        if (!ok) break;
        const bool more = g + 1 < n_kv;
        const uint32_t full = bar(kBarPairFull + g % kPairBars);
        mbar_expect_tx(full, more ? 2 * kTileBytes : kTileBytes);
        load_tile(&tm_v, 2 * g + 1, g, full);
        if (more) load_tile(&tm_k, 2 * g + 2, g + 1, full);
        issued = g + 1;
      }
      if (!ok) {
        // leave no copy in flight: wait (bounded) for the tiles already requested
        const long long t0 = clock64();
        while (!mbar_try_wait(bar(kBarK0Full), 0) && clock64() - t0 < kWaitBudgetCycles) {
        }
        for (int g = (issued > kPairBars ? issued - kPairBars : 0); g < issued; ++g) {
          const long long t1 = clock64();
          while (!mbar_try_wait(bar(kBarPairFull + g % kPairBars), (g / kPairBars) & 1) &&
                 clock64() - t1 < kWaitBudgetCycles) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const int n_stage = two_tiles ? 2 : 1;
      const uint32_t sq[2] = {base + kSmemQ, base + kSmemQ + kTileBytes};
      const uint32_t tS[2] = {tmem + kColS, tmem + kColS + 128};
      const uint32_t tO[2] = {tmem + kColO, tmem + kColO + 128};
      auto slot_addr = [&](int it) { return base + kSmemKV + (it % kSlots) * kTileBytes; };
      bool ok = mbar_wait(bar(kBarK0Full), 0, abort_flag, p.status, WAIT_KV_FULL);
      for (int s = 0; s < n_stage && ok; ++s) {
        ok = mbar_wait(bar(kBarQFull + s), 0, abort_flag, p.status, WAIT_Q_FULL);
        if (!ok) break;
        tc_fence_after();
        issue_qk(tS[s], sq[s], slot_addr(0));
        umma_commit(bar(kBarSFull + s));
      }
      // step j: O += P_j V_j and S = Q K_{j+1}^T for each query tile; V_j and K_{j+1} are pair j of the ring
      int slot_v = 1 % kSlots, slot_k = 2 % kSlots, pair_bar = 0, pair_par = 0;
      for (int j = 0; j < n_kv && ok; ++j) {
        const bool more = j + 1 < n_kv;
        const uint32_t sv = base + kSmemKV + slot_v * kTileBytes, sk = base + kSmemKV + slot_k * kTileBytes;
        for (int s = 0; s < n_stage && ok; ++s) {
          stamp(j, s * 6 + 0);
          ok = mbar_wait(bar(kBarPHalf + s), j & 1, abort_flag, p.status, WAIT_P_FULL);
          stamp(j, s * 6 + 1);
          if (ok && s == 0) ok = mbar_wait(bar(kBarPairFull + pair_bar), pair_par, abort_flag, p.status, WAIT_KV_FULL);
          if (!ok) break;
          tc_fence_after();
          issue_pv(tO[s], tS[s], sv, j > 0, 0, 4);
          stamp(j, s * 6 + 2);
          ok = mbar_wait(bar(kBarPFull + s), j & 1, abort_flag, p.status, WAIT_P_FULL);
          stamp(j, s * 6 + 3);
          if (!ok) break;
          tc_fence_after();
          issue_pv(tO[s], tS[s], sv, true, 4, 8);
          if (more) {
            issue_qk(tS[s], sq[s], sk);
            stamp(j, s * 6 + 4);
            umma_commit(bar(kBarSFull + s));
          } else {
            umma_commit(bar(kBarOFull + s));
          }
          stamp(j, s * 6 + 5);
        }
        if (ok) umma_commit(bar(kBarPairDone + pair_bar));
        slot_v = slot_v + 2 >= kSlots ? slot_v + 2 - kSlots : slot_v + 2;
        slot_k = slot_k + 2 >= kSlots ? slot_k + 2 - kSlots : slot_k + 2;
        if (++pair_bar == kPairBars) {
          pair_bar = 0;
          pair_par ^= 1;
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + epilogue
    const int stage = (warp - 4) >> 2;
    if (stage == 0 || two_tiles) {
      const int quad = warp & 3;
      const int row = quad * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
      const uint32_t tS = tmem + lane_base + kColS + stage * 128;
      const uint32_t tO = tmem + lane_base + kColO + stage * 128;
      const float scale = p.scale_log2;
      float m_used = -INFINITY;
      float l = 0.f;
      bool ok = true;
      for (int j = 0; j < n_kv; ++j) {
        if (row == 0) stamp(j, 12 + stage * 6 + 0);
        ok = mbar_wait(bar(kBarSFull + stage), j & 1, abort_flag, p.status, WAIT_S_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (row == 0) stamp(j, 12 + stage * 6 + 1);
        tc_fence_after();
        uint32_t s[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, s[c]);
        tmem_wait_ld();
        const int valid = seq_len - (j0 + j) * kBN;
        if (valid < kBN) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i >= valid) s[c][i] = 0xFF800000u;  // -inf
          // The V rows behind those keys lie inside the cache, so the TMA did not zero-fill them and they
          // may hold anything, NaN included; P is 0 there, but 0 x NaN would poison the whole output row.
          // Query tile 0 clears them in shared memory before it reports P (tile 1's P V is issued later).
          if (stage == 0) {
            const int it_v = 2 * j + 1;
            ok = mbar_wait(bar(kBarPairFull + j % kPairBars), (j / kPairBars) & 1, abort_flag, p.status, WAIT_KV_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (row >= valid) {
              uint8_t* vrow = gbase + kSmemKV + (it_v % kSlots) * kTileBytes + row * 128;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                *reinterpret_cast<uint4*>(vrow + 16 * i) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(vrow + kHalfTile + 16 * i) = make_uint4(0u, 0u, 0u, 0u);
              }
            }
            fence_proxy_async_smem();
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx0 = fmaxf(mx0, __uint_as_float(s[c][i]));
            mx1 = fmaxf(mx1, __uint_as_float(s[c][i + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(s[c][i + 2]));
            mx3 = fmaxf(mx3, __uint_as_float(s[c][i + 3]));
          }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale;
        if (row == 0) stamp(j, 12 + stage * 6 + 2);
        if (j == 0) {
          m_used = mx;  // tile 0 always has a valid column, so mx is finite
        } else {
          const bool grow = mx > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, grow)) {
            const float m_new = grow ? mx : m_used;
            const float alpha = ex2_approx(m_used - m_new);
            m_used = m_new;
            l *= alpha;
            // O of this stage is idle here: P V of the previous kv tile completed before S arrived
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(tO + c * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + c * 32, o);
            }
          }
        }
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(s[c][2 * i]), scale, -m_used));
            const float p1 = ex2_approx(fmaf(__uint_as_float(s[c][2 * i + 1]), scale, -m_used));
            sum0 += p0;
            sum1 += p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st16(tS + c * 16, pk);
          if (c == 1) {  // the first 64 keys of P are complete: their share of P V can start
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(kBarPHalf + stage));
            if (row == 0) stamp(j, 12 + stage * 6 + 3);
          }
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(kBarPFull + stage));
        if (row == 0) stamp(j, 12 + stage * 6 + 4);
        l += sum0 + sum1;
      }
      if (ok) {
        ok = mbar_wait(bar(kBarOFull + stage), 0, abort_flag, p.status, WAIT_O_FULL);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok && part < 0) {
        tc_fence_after();
        const float inv = 1.f / l;
        const int q_row = q0 + stage * kBM + row;
        __nv_bfloat16* op = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(b) * p.out_stride_row +
                            static_cast<int64_t>(q_row) * p.out_stride_tok +
                            static_cast<int64_t>(h) * p.out_stride_head;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
          if (q_row < p.q_tokens) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
              *reinterpret_cast<uint4*>(op + c * 32 + i * 8) = v;
            }
          }
        }
      } else if (ok) {
        // partial result of one key range: unnormalised accumulator, running max and sum
        tc_fence_after();
        const int slot = (tile - p.n_full) * p.split + part;
        float* po = p.part_o + (static_cast<size_t>(slot) * 2 + stage) * (kBM * kHD) + row * kHD;
        float* pml = p.part_ml + (static_cast<size_t>(slot) * 2 + stage) * (2 * kBM);
        pml[row] = m_used;
        pml[kBM + row] = l;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<uint4*>(po + c * 32 + i * 4) = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// -------------------------------------------------------------------------------------------
// Self-test of the two contractions in isolation (128 threads, one CTA).
// -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_v, const __nv_bfloat16* __restrict__ pmat,
                     float* __restrict__ s_out, float* __restrict__ o_out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t sA = base, sB = base + kTileBytes, sV = base + 2 * kTileBytes;
  const uint32_t bar0 = base + 3 * kTileBytes;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 3 * kTileBytes + 64);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + 3 * kTileBytes + 68);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 3; ++i) mbar_init(bar0 + 8 * i, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  const int row = warp * 32 + lane;

  if (threadIdx.x == 0) {
    mbar_expect_tx(bar0, 3 * kTileBytes);
    tma_load_2d(sA, &tm_a, bar0, 0, 0);
    tma_load_2d(sA + kHalfTile, &tm_a, bar0, 64, 0);
    tma_load_2d(sB, &tm_b, bar0, 0, 0);
    tma_load_2d(sB + kHalfTile, &tm_b, bar0, 64, 0);
    tma_load_2d(sV, &tm_v, bar0, 0, 0);
    tma_load_2d(sV + kHalfTile, &tm_v, bar0, 64, 0);
    if (mbar_wait(bar0, 0, abort_flag, status, WAIT_PROBE)) {
      tc_fence_after();
      issue_qk(tS, sA, sB);
      umma_commit(bar0 + 8);
    }
  }
  bool ok = mbar_wait(bar0 + 8, 0, abort_flag, status, WAIT_PROBE);
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tS + lane_base + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) s_out[row * 128 + c * 32 + i] = __uint_as_float(r[i]);
    }
    // P row -> TMEM columns [0,64) of S, two bf16 per 32-bit column (even column in the low half)
    const uint32_t* prow = reinterpret_cast<const uint32_t*>(pmat + row * 128);
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = prow[c * 32 + i];
      tmem_st32(tS + lane_base + c * 32, r);
    }
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag) {
    tc_fence_after();
    issue_pv(tO, tS, sV, false);
    umma_commit(bar0 + 16);
  }
  ok = mbar_wait(bar0 + 16, 0, abort_flag, status, WAIT_PROBE);
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tO + lane_base + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_out[row * 128 + c * 32 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 256);
  }
}

// One warp waits on a barrier that nobody completes; the wait gives up after `budget` cycles and
// reports like every other bounded wait in this library.
__global__ void __launch_bounds__(32, 1) wait_timeout_selftest_kernel(int* status, long long budget) {
  __shared__ __align__(8) uint64_t never_completed;
  __shared__ int abort_word;
  const uint32_t bar = smem_u32(&never_completed);
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) mbar_wait(bar, 0, abort_flag, status, WAIT_PROBE, budget);
  __syncwarp();
  // the other lanes take the same exit the kernels' roles take: they see the raised flag at once
  if (threadIdx.x != 0) mbar_wait(bar, 0, abort_flag, nullptr, WAIT_PROBE, budget);
}

// Measurement aid (SDV2_ATTN_TRACE with bit 8): every CTA issues runs of 64 MMAs of one kind back to back
// on real tiles and records the cycles from the first issue to the completion of the last one.
//   0 SS K-major N=128   1 TS + MN-major B N=128   2 SS, MN-major B   3 kinds 0 and 1 alternating by fours
//   4 SS K-major N=64    5 SS K-major N=256 (B rows past 128 are whatever follows the tile)
__global__ void __launch_bounds__(128, 1)
umma_rate_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (base - raw);
  const uint32_t sQ = base, sK = base + kTileBytes, sK2 = base + 2 * kTileBytes, sV = base + 3 * kTileBytes;
  const uint32_t bar0 = base + 4 * kTileBytes;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + 4 * kTileBytes + 64);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + 4 * kTileBytes + 68);
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar0, 1);
    mbar_init(bar0 + 8, 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (threadIdx.x == 0) {
    const int h = blockIdx.x % p.heads;
    mbar_expect_tx(bar0, 4 * kTileBytes);
    for (int half = 0; half < 2; ++half) {
      tma_load_4d(sQ + half * kHalfTile, &tm_q, bar0, 64 * half, h, 0, 0);
      tma_load_4d(sK + half * kHalfTile, &tm_k, bar0, 64 * half, h, 0, 0);
      tma_load_4d(sK2 + half * kHalfTile, &tm_k, bar0, 64 * half, h, 128, 0);
      tma_load_4d(sV + half * kHalfTile, &tm_v, bar0, 64 * half, h, 0, 0);
    }
    bool ok = mbar_wait(bar0, 0, abort_flag, p.status, WAIT_PROBE);
    constexpr uint32_t kIdesc64 = umma_idesc_bf16(kBM, 64, false, false);
    constexpr uint32_t kIdesc256 = umma_idesc_bf16(kBM, 256, false, false);
    uint32_t parity = 0;
    for (int v = 0; v < 8 && ok; ++v) {
      tc_fence_after();
      const long long t0 = clock64();
      for (int rep = 0; rep < 8; ++rep) {
        if (v == 0) issue_qk(tmem + kColS, sQ, sK);
        if (v == 1) issue_pv(tmem + kColO, tmem + kColS + 128, sV, rep > 0);
        if (v == 2) issue_pv(tmem + kColO, 0, sV, rep > 0, 0, 8, true, sQ);
        if (v == 3) {
          issue_pv(tmem + kColO, tmem + kColS + 128, sV, rep > 0, 0, 4);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t off = (k & 3) * 32;
            umma_ss(tmem + kColS, umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024), kIdescQK,
                    k > 0 ? 1u : 0u);
          }
        }
        if (v == 6 && rep < 4) {  // 6: whole P V then whole Q K^T, as the kernel orders them
          issue_pv(tmem + kColO, tmem + kColS + 128, sV, rep > 0);
          issue_qk(tmem + kColS, sQ, sK);
        }
        if (v == 7) issue_qk(tmem + kColS + (rep & 1) * 128, sQ, sK);  // 7: kind 0, two accumulators in turn
        if (v == 4 || v == 5) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * kHalfTile + (k & 3) * 32;
            umma_ss(tmem + kColS, umma_smem_desc(sQ + off, 16, 1024), umma_smem_desc(sK + off, 16, 1024),
                    v == 4 ? kIdesc64 : kIdesc256, k > 0 ? 1u : 0u);
          }
        }
      }
      umma_commit(bar0 + 8);
      ok = mbar_wait(bar0 + 8, parity, abort_flag, p.status, WAIT_PROBE);
      parity ^= 1;
      const long long t1 = clock64();
      if (blockIdx.x < 16) p.trace[blockIdx.x * 8 + v] = t1 - t0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace attn

// Merge the partial results of the split tail tiles.  Block = (tail tile, query tile, group of 32
// rows); 256 threads = 32 rows x 8 column groups of 16, so the 8 threads of a row read its 512
// bytes of each partial accumulator contiguously.  out = sum_k 2^(m_k - m) O_k / sum_k 2^(m_k - m) l_k.
__global__ void __launch_bounds__(256) attn_combine_kernel(const __grid_constant__ AttnParams p) {
  using namespace attn;
  const int tail = blockIdx.x, stage = blockIdx.y;
  const int row = blockIdx.z * 32 + (threadIdx.x >> 3);
  const int c0 = (threadIdx.x & 7) * 16;
  const int tile = p.n_full + tail;
  const int pt = tile % p.pair_tiles;
  const int hb = tile / p.pair_tiles;
  const int h = hb % p.heads;
  const int b = hb / p.heads;
  const int q_row = pt * (2 * kBM) + stage * kBM + row;
  if (q_row >= p.q_tokens) return;
  const float* ml = p.part_ml + (static_cast<size_t>(tail) * p.split * 2 + stage) * (2 * kBM);
  const float* po = p.part_o + (static_cast<size_t>(tail) * p.split * 2 + stage) * (kBM * kHD) + row * kHD + c0;
  const size_t ml_step = 2 * 2 * kBM, po_step = static_cast<size_t>(2) * kBM * kHD;
  float m = -INFINITY;
  for (int k = 0; k < p.split; ++k) m = fmaxf(m, ml[k * ml_step + row]);
  float l = 0.f;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (int k = 0; k < p.split; ++k) {
    const float w = exp2f(ml[k * ml_step + row] - m);
    l += w * ml[k * ml_step + kBM + row];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 a = *reinterpret_cast<const float4*>(po + k * po_step + 4 * i);
      acc[4 * i + 0] += w * a.x; acc[4 * i + 1] += w * a.y; acc[4 * i + 2] += w * a.z; acc[4 * i + 3] += w * a.w;
    }
  }
  const float inv = 1.f / l;
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(b) * p.out_stride_row +
                      static_cast<int64_t>(q_row) * p.out_stride_tok + static_cast<int64_t>(h) * p.out_stride_head + c0;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 v;
    v.x = pack_bf16x2(acc[8 * i + 0] * inv, acc[8 * i + 1] * inv);
    v.y = pack_bf16x2(acc[8 * i + 2] * inv, acc[8 * i + 3] * inv);
    v.z = pack_bf16x2(acc[8 * i + 4] * inv, acc[8 * i + 5] * inv);
    v.w = pack_bf16x2(acc[8 * i + 6] * inv, acc[8 * i + 7] * inv);
    *reinterpret_cast<uint4*>(op + 8 * i) = v;
  }
}

cudaError_t launch_attn_tcgen05(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v,
                                const AttnParams& p_in, cudaStream_t stream) {
  static DynamicSmemGrant smem_grant, smem_grant_trace;
  AttnParams p = p_in;
  DeviceInfo di;
  cudaError_t e = device_info(&di);
  if (e == cudaSuccess)
    e = p.trace != nullptr
            ? smem_grant_trace.ensure(attn::attn_fwd_kernel<true>, static_cast<int>(attn::kSmemBytes), di.device)
            : smem_grant.ensure(attn::attn_fwd_kernel<false>, static_cast<int>(attn::kSmemBytes), di.device);
  if (e != cudaSuccess) return e;
  if (p.trace != nullptr && (p.trace_mode & 256)) {
    static DynamicSmemGrant rate_grant;
    const int smem = 4 * attn::kTileBytes + 128 + 1024;
    e = rate_grant.ensure(attn::umma_rate_kernel, smem, di.device);
    if (e != cudaSuccess) return e;
    attn::umma_rate_kernel<<<di.sms, 128, smem, stream>>>(tm_q, tm_k, tm_v, p);
    return cudaGetLastError();
  }
  p.pair_tiles = (p.q_tokens + 2 * attn::kBM - 1) / (2 * attn::kBM);
  const int64_t n_tiles = static_cast<int64_t>(p.pair_tiles) * p.heads * p.rows;
  if (n_tiles > 0x7FFFFFFFLL) return cudaErrorInvalidValue;
  int min_kv = 0x7FFFFFFF;
  for (int b = 0; b < p.rows; ++b) min_kv = min(min_kv, (p.seq_lens[b] + attn::kBN - 1) / attn::kBN);
  // whole tiles keep the head-major order; the tiles of the last, partly filled wave are cut into key ranges
  p.split = attn_tail_split(n_tiles, di.sms, min_kv, p.part_o != nullptr, &p.n_tail);
  p.n_full = static_cast<int>(n_tiles) - p.n_tail;
  const unsigned grid = static_cast<unsigned>(p.n_full + p.n_tail * p.split);
  if (p.trace != nullptr)
    attn::attn_fwd_kernel<true><<<grid, attn::kThreads, attn::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
  else
    attn::attn_fwd_kernel<false><<<grid, attn::kThreads, attn::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, p);
  e = cudaGetLastError();
  if (e != cudaSuccess || p.n_tail == 0) return e;
  attn_combine_kernel<<<dim3(p.n_tail, 2, attn::kBM / 32), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_umma_selftest(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_v,
                                 const void* p_dev, float* s_out, float* o_out, int* status,
                                 cudaStream_t stream) {
  static DynamicSmemGrant smem_grant;
  const int smem = 3 * attn::kTileBytes + 128 + 1024;
  DeviceInfo di;
  cudaError_t attr = device_info(&di);
  if (attr == cudaSuccess) attr = smem_grant.ensure(attn::umma_selftest_kernel, smem, di.device);
  if (attr != cudaSuccess) return attr;
  attn::umma_selftest_kernel<<<1, 128, smem, stream>>>(tm_a, tm_b, tm_v,
                                                      static_cast<const __nv_bfloat16*>(p_dev), s_out, o_out,
                                                      status);
  return cudaGetLastError();
}

cudaError_t launch_wait_timeout_selftest(int* status, long long budget_cycles, cudaStream_t stream) {
  attn::wait_timeout_selftest_kernel<<<1, 32, 0, stream>>>(status, budget_cycles);
  return cudaGetLastError();
}

}  // namespace sdv2
