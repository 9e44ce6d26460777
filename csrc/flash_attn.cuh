// Fused attention forward on the 5th-generation tensor cores: O = softmax(scale * Q K^T [+ causal mask]) V.
//
// One CTA owns 128 query rows of one (batch, head) and walks the keys in tiles of 128:
//
//   warp 8     TMA producer: Q once, then K and V tiles into rings of 2 (D = 128) or 4 (D = 64) stages, 128-byte-swizzled 64-wide blocks
//   warp 9     MMA issuer:   S_j = Q K_j^T   -> TMEM columns [0,256), double buffered
//                            O  += P_j V_j   -> TMEM columns [256, 256 + D), accumulated across the key tiles
//   warps 0-7  softmax:      TMEM lane r holds query row r; warps w and w+4 share the 32 rows of lane quadrant w and
//                            take 64 of the 128 key columns each, so every scheduler has two resident warps to hide the
//                            TMEM-load, MUFU and shared-memory latencies of the other.  A thread reads its half of S_j
//                            once, exponentiates against a *reference* maximum, writes its half of P_j as bf16 into the
//                            swizzled K-major operand layout in shared memory and keeps a partial running sum.  The two
//                            halves of a row agree on the reference through one bf16 exchange per tile.
//
// Lazy rescaling.  The reference maximum of a row only moves when the row maximum of a tile exceeds it by more than
// 2^8; bf16 and fp32 share their exponent range, so exponentials up to 2^8 (and, before a redo is forced, 2^64) are
// exact enough and cannot overflow.  While the reference stays put the accumulator in TMEM needs no correction at
// all; when it moves, the warp reads its 32 accumulator rows, scales them and writes them back (tcgen05.ld / st)
// before it releases P_j, i.e. strictly between the products of tiles j-1 and j.  A tile whose maximum exceeds the
// reference by more than 2^64 (only possible with pathological inputs; always the case for the first tile, whose
// reference is -inf) is redone against its own maximum while S_j is still in TMEM.
//
// S_{j+1} is issued before P_j is waited for, so the QK^T product of the next tile overlaps the softmax of this one,
// and the product P_j V_j overlaps the softmax of tile j+1.  Every reuse of a TMEM or shared-memory buffer is ordered
// by the p_full / o_full barriers that the loops wait on anyway (see the comments at the waits).
//
// V is consumed either in its natural [keys, D] layout as an MN-major B operand (VT = false) or from a pre-transposed
// [D, keys] copy as a K-major operand (VT = true).  Rows of K / V beyond the sequence read as zero through TMA and are
// masked to -inf before the softmax.  All barrier waits are bounded; a wait that runs out records an error code,
// releases the other waiters of the CTA, and the CTA still frees its TMEM and returns.
#pragma once
#include <cuda_bf16.h>
#include <math.h>

#include "common.cuh"
#include "tmap.cuh"

namespace pnm {

struct FlashArgs {
  CUtensorMap tmQ, tmK, tmV;
  __nv_bfloat16* out;  // [BH, Sq, D]
  float* lse;          // [BH, Sq] natural-log sum of exponentials, may be null
  int Sq, Skv, n_qtiles;
  float scale_log2;    // softmax scale * log2(e)
  int causal;
  int* err;
};

constexpr int kFaThreads = 320;
constexpr int kFaPolyMask = 0;   // bit i set: exponential i of every eight goes to the FMA-pipe polynomial (measured slower: the FMA pipe is the busier one)
constexpr int kFaBarBytes = 256 + 1024;   // barriers, then the 1 KB exchange area of the row halves

template <int D>
__host__ __device__ constexpr int flash_kv_stages() { return D == 64 ? 4 : 2; }   // 16 KB tiles at D = 64: a deeper ring hides the L2 latency

template <int D>
constexpr int flash_smem_bytes() { return 1024 + (1 + 2 * flash_kv_stages<D>()) * (128 * D * 2) + 2 * (128 * 128 * 2) + kFaBarBytes; }

// Bounded wait that never raises the abort flag: used to let copies in flight land before an aborted CTA leaves.
__device__ __forceinline__ void mbar_drain(uint64_t* bar, uint32_t parity) {
  const unsigned long long t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (globaltimer_ns() - t0 > kWaitBudgetNs) break;
  }
}

template <int D, bool VT, bool PTM>
__global__ void __launch_bounds__(kFaThreads, 1) flash_fwd_kernel(const __grid_constant__ FlashArgs g) {
  static_assert(D == 64 || D == 128, "head dimension 64 or 128");
  constexpr int KB = D / 64;
  constexpr int ST = flash_kv_stages<D>();   // K / V ring depth
  constexpr int TILE = 128 * D * 2;   // bytes of a Q, K or V tile
  constexpr int PT = 128 * 128 * 2;   // bytes of a P tile
  constexpr int BLK = 128 * 128;      // bytes of a [128 rows x 64] block
  extern __shared__ uint8_t fa_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = base;
  uint8_t* sK = sQ + TILE;
  uint8_t* sV = sK + ST * TILE;
  uint8_t* sP = sV + ST * TILE;
  uint64_t* bar = reinterpret_cast<uint64_t*>(sP + 2 * PT);
  uint64_t* q_full = bar;
  uint64_t* k_full = bar + 1;    // [4]
  uint64_t* k_empty = bar + 5;   // [4]
  uint64_t* v_full = bar + 9;    // [4]
  uint64_t* v_empty = bar + 13;  // [4]
  uint64_t* s_full = bar + 17;   // [2]
  uint64_t* p_full = bar + 19;   // [2]
  uint64_t* o_full = bar + 21;
  uint64_t* xbar = bar + 22;     // [4] one per lane quadrant: the two warps of a row group meet here
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 26);
  uint8_t* xchg = reinterpret_cast<uint8_t*>(bar) + 256;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x / g.n_qtiles;
  const int qt = g.n_qtiles - 1 - (blockIdx.x % g.n_qtiles);   // long (late) causal rows first
  const int q0 = qt * 128;
  int T = (g.Skv + 127) >> 7;
  if (g.causal) T = min(T, qt + 1);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 8);   // one arrival per softmax warp
    }
    mbar_init(o_full, 1);
    for (int w = 0; w < 4; ++w) mbar_init(&xbar[w], 2);
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&g.tmQ);
    tma_prefetch_desc(&g.tmK);
    tma_prefetch_desc(&g.tmV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE);
      for (int kb = 0; kb < KB; ++kb) tma_load_3d(sQ + kb * BLK, &g.tmQ, q_full, kb * 64, q0, bh);
      int issued = 0;
      for (int j = 0; j < T; ++j) {
        const int s = j % ST;
        const uint32_t ph = (j / ST) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag, g.err, ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&k_full[s], TILE);
        for (int kb = 0; kb < KB; ++kb) tma_load_3d(sK + s * TILE + kb * BLK, &g.tmK, &k_full[s], kb * 64, j * 128, bh);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag, g.err, ERR_WAIT_EMPTY)) { issued = -(j + 1); break; }
        mbar_expect_tx(&v_full[s], TILE);
        if (VT) {
          for (int kb = 0; kb < 2; ++kb)
            tma_load_3d(sV + s * TILE + kb * (D * 128), &g.tmV, &v_full[s], j * 128 + kb * 64, 0, bh);
        } else {
          for (int kb = 0; kb < KB; ++kb)
            tma_load_3d(sV + s * TILE + kb * BLK, &g.tmV, &v_full[s], kb * 64, j * 128, bh);
        }
        issued = j + 1;
      }
      if (*abort_flag) {
        // let the copies that were issued land before the CTA's shared memory goes away
        mbar_drain(q_full, 0);
        const int nk = issued < 0 ? -issued : issued, nv = issued < 0 ? -issued - 1 : issued;
        for (int j = max(nk - ST, 0); j < nk; ++j) mbar_drain(&k_full[j % ST], (j / ST) & 1);
        for (int j = max(nv - ST, 0); j < nv; ++j) mbar_drain(&v_full[j % ST], (j / ST) & 1);
      }
    }
  } else if (warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, false, !VT);
      bool ok = mbar_wait(q_full, 0, abort_flag, g.err, ERR_WAIT_FULL);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % ST;
        if (!mbar_wait(&k_full[s], (j / ST) & 1, abort_flag, g.err, ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t d = tmem_base + (j & 1) * 128;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          const uint64_t ad = make_smem_desc(smem_u32(sQ + kb * BLK), 16, 1024, 2);
          const uint64_t bd = make_smem_desc(smem_u32(sK + s * TILE + kb * BLK), 16, 1024, 2);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(d, ad + 2 * k, bd + 2 * k, idesc_s, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[s]);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok && T > 0) ok = issue_qk(0);
      for (int j = 0; ok && j < T; ++j) {
        // S buffer (j+1)&1 was last read by the softmax of tile j-1, which ended before p_full of tile j-1 completed
        if (j + 1 < T && !issue_qk(j + 1)) { ok = false; break; }
        const int s = j & 1, sv = j % ST;
        const uint32_t ph = (j >> 1) & 1;
        // p_full of tile j also means: the product of tile j-1 has completed (every thread waits for o_full of tile
        // j-1 before it arrives) and any correction of the accumulator has been written back
        if (!mbar_wait(&p_full[s], ph, abort_flag, g.err, ERR_WAIT_AUX)) { ok = false; break; }
        if (!mbar_wait(&v_full[sv], (j / ST) & 1, abort_flag, g.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d = tmem_base + 256;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint64_t bd;
          if (VT) bd = make_smem_desc(smem_u32(sV + sv * TILE + (k >> 2) * (D * 128)), 16, 1024, 2) + 2 * (k & 3);
          else bd = make_smem_desc(smem_u32(sV + sv * TILE + k * 2048), BLK, 1024, 2);   // 16 key rows per step
          if (PTM) {
            // P_j sits in tensor memory (columns 384 + 64 s ...), 8 packed columns per 16 keys
            umma_f16_ts(d, tmem_base + 384 + s * 64 + k * 8, bd, idesc_o, (j | k) != 0 ? 1u : 0u);
          } else {
            const uint64_t ad = make_smem_desc(smem_u32(sP + s * PT + (k >> 2) * BLK), 16, 1024, 2) + 2 * (k & 3);
            umma_f16(d, ad, bd, idesc_o, (j | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(&v_empty[sv]);
        umma_commit(o_full);
      }
    }
  } else {
    // ------------------------------------------------------------- softmax rows
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
    const float c = g.scale_log2;
    __nv_bfloat16* xmax = reinterpret_cast<__nv_bfloat16*>(xchg);   // [tile parity][half][row]
    float* xsum = reinterpret_cast<float*>(xchg);                    // [half][row], after the last tile
    float ref = -INFINITY;    // reference maximum of the previous tile (what the accumulator and l are relative to)
    float next = -INFINITY;   // reference chosen for the coming tile
    float l = 0.f;            // this half's part of the row sum
    bool ok = true;
    constexpr int OC = D / 64;   // 32-column chunks of the accumulator per half

    // the two warps of a row group meet: publish (done by the caller), one arrival per warp, bounded wait
    auto meet = [&](int phase) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(&xbar[quad]);
      return __all_sync(0xffffffffu, mbar_wait(&xbar[quad], phase & 1, abort_flag, g.err, ERR_WAIT_AUX));
    };

    for (int j = 0; j < T; ++j) {
      const int s = j & 1;
      // the TMEM loads below are warp-collective: the warp leaves together or not at all
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, g.err, ERR_WAIT_TMEM_FULL))) { ok = false; break; }
      tc_fence_after();
      const bool edge = (j * 128 + 128 > g.Skv) || (g.causal && j * 128 + 127 > q0);
      int lim = g.Skv - j * 128;
      if (g.causal) lim = min(lim, q0 + row - j * 128 + 1);
      lim -= half * 64;   // in this half's column numbering
      float v[64];
      tmem_ld32(lane_addr + s * 128 + half * 64, v);
      tmem_ld32(lane_addr + s * 128 + half * 64 + 32, v + 32);
      tmem_ld_wait();
      if (edge) {
#pragma unroll
        for (int i = 0; i < 64; ++i) if (i >= lim) v[i] = -INFINITY;
      }
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        m0 = fmaxf(m0, v[i]);
        m1 = fmaxf(m1, v[i + 1]);
        m2 = fmaxf(m2, v[i + 2]);
        m3 = fmaxf(m3, v[i + 3]);
      }
      // the maximum only serves as a reference, so the halves exchange it rounded up to bf16
      const __nv_bfloat16 mine = __float2bfloat16_ru(fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * c);
      xmax[(s * 2 + half) * 128 + row] = mine;
      if (!meet(j)) { ok = false; break; }
      const float tile_max = fmaxf(__bfloat162float(mine), __bfloat162float(xmax[(s * 2 + (half ^ 1)) * 128 + row]));
      // first tile, or a jump of more than 2^64 somewhere in the row group: take the tile's own maximum as reference
      if (__any_sync(0xffffffffu, tile_max - next > 64.f)) next = fmaxf(next, tile_max);
      const float use = (next == -INFINITY) ? 0.f : next;
      const float alpha = ex2_fast(ref - use);   // 0 for the first tile, 1 while the reference stays put
      float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
      // P buffer s was last read by the product of tile j-2, whose o_full this thread waited for in iteration j-1
      uint8_t* prow = sP + s * PT + half * BLK + row * 128;
      uint32_t packed[32];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          // the special-function unit (16 results per clock and SM) is the busiest pipe of the softmax: every other
          // exponential is evaluated by a cubic on the FMA pipe instead
          const float a = fmaf(v[q * 8 + i], c, -use);
          e[i] = ((kFaPolyMask >> i) & 1) ? ex2_poly(a) : ex2_fast(a);
        }
        rs0 += e[0] + e[4];
        rs1 += e[1] + e[5];
        rs2 += e[2] + e[6];
        rs3 += e[3] + e[7];
        uint4 u;
        u.x = pack_bf16x2(e[0], e[1]);
        u.y = pack_bf16x2(e[2], e[3]);
        u.z = pack_bf16x2(e[4], e[5]);
        u.w = pack_bf16x2(e[6], e[7]);
        if (PTM) {
          packed[q * 4 + 0] = u.x;
          packed[q * 4 + 1] = u.y;
          packed[q * 4 + 2] = u.z;
          packed[q * 4 + 3] = u.w;
        } else {
          *reinterpret_cast<uint4*>(prow + ((q ^ (row & 7)) << 4)) = u;
        }
      }
      if (PTM) {
        // this half's 64 probabilities = 32 packed columns of the P buffer of tile parity s
        tmem_st32(lane_addr + 384 + s * 64 + half * 32, reinterpret_cast<const float*>(packed));
        tmem_st_wait();
      }
      l = fmaf(l, alpha, (rs0 + rs1) + (rs2 + rs3));
      if (j > 0) {
        // product of tile j-1 done: until the arrive below the accumulator is free to touch
        if (!__all_sync(0xffffffffu, mbar_wait(o_full, (j - 1) & 1, abort_flag, g.err, ERR_WAIT_TMEM_FULL))) { ok = false; break; }
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < OC; ++cc) {
            float o[32];
            const uint32_t at = lane_addr + 256 + half * (D / 2) + cc * 32;
            tmem_ld32(at, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_st32(at, o);
          }
          tmem_st_wait();
        }
      }
      if (!PTM) fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
      ref = use;
      next = (tile_max - use > 8.f) ? tile_max : use;
    }
    if (ok && T > 0) ok = __all_sync(0xffffffffu, mbar_wait(o_full, (T - 1) & 1, abort_flag, g.err, ERR_WAIT_TMEM_FULL));
    if (ok) {
      // every softmax warp has arrived on p_full of the last tile, i.e. is past its last read of the exchange area
      xsum[half * 128 + row] = l;
      ok = meet(T);
    }
    if (ok) {
      tc_fence_after();
      const float lt = l + xsum[(half ^ 1) * 128 + row];
      const bool live = q0 + row < g.Sq;
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      __nv_bfloat16* dst = g.out + (size_t(bh) * g.Sq + q0 + row) * D + half * (D / 2);
#pragma unroll
      for (int cc = 0; cc < OC; ++cc) {
        float o[32];
        tmem_ld32(lane_addr + 256 + half * (D / 2) + cc * 32, o);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 u;
            u.x = pack_bf16x2(o[i + 0] * inv, o[i + 1] * inv);
            u.y = pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv);
            u.z = pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv);
            u.w = pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv);
            *reinterpret_cast<uint4*>(dst + cc * 32 + i) = u;
          }
        }
      }
      if (live && half == 0 && g.lse)
        g.lse[size_t(bh) * g.Sq + q0 + row] = lt > 0.f ? (ref + log2f(lt)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

struct FlashCall {
  const void* q; const void* k; const void* v; void* out; float* lse;
  int BH, Sq, Skv, ldv;   // ldv: row stride of the transposed V copy (elements), unused otherwise
  float scale;
  int causal;
};

template <int D, bool VT, bool PTM>
int launch_flash_fwd(const FlashCall& c, int* err, cudaStream_t st) {
  FlashArgs a;
  if (make_tmap_3d_b16(&a.tmQ, c.q, c.BH, c.Sq, D, D, uint64_t(c.Sq) * D, 128)) return -2;
  if (make_tmap_3d_b16(&a.tmK, c.k, c.BH, c.Skv, D, D, uint64_t(c.Skv) * D, 128)) return -2;
  if (VT) {
    if (make_tmap_3d_b16(&a.tmV, c.v, c.BH, D, c.Skv, c.ldv, uint64_t(c.ldv) * D, D)) return -2;
  } else {
    if (make_tmap_3d_b16(&a.tmV, c.v, c.BH, c.Skv, D, D, uint64_t(c.Skv) * D, 128)) return -2;
  }
  a.out = reinterpret_cast<__nv_bfloat16*>(c.out);
  a.lse = c.lse;
  a.Sq = c.Sq;
  a.Skv = c.Skv;
  a.n_qtiles = (c.Sq + 127) / 128;
  a.scale_log2 = c.scale * 1.4426950408889634f;
  a.causal = c.causal;
  a.err = err;
  constexpr int smem = flash_smem_bytes<D>();
  auto kern = flash_fwd_kernel<D, VT, PTM>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -3;
  const long long ctas = (long long)a.n_qtiles * c.BH;
  if (ctas <= 0 || ctas > 0x7fffffffLL) return -1;
  kern<<<(unsigned)ctas, kFaThreads, smem, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace pnm
