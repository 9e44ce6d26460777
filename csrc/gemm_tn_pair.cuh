// C[M,N] = epilogue( A[M,K] * B[N,K]^T ) on CTA PAIRS: one 256 x BN output tile (BN = 256 or 128) per cluster of two
// CTAs, computed by tcgen05.mma.cta_group::2.  A is a row-major matrix or, in convolution mode, the shifted windows of a
// channels-last image (implicit GEMM, the same 8 x 16 pixel tiles and tap-major K order as the single-CTA kernel).
//
// Why: the single-CTA kernel (gemm_tn.cuh) loads (128 + 256) x 64 operand elements per 128 x 256 x 64 block of products,
// 85 FLOP per byte brought from L2 into shared memory.  For compute-bound shapes (K >= 512) that traffic, not the tensor
// pipe, sets the pace: the 128 x 128 and the 128 x 256 tile both stop near the same L2 -> SM bandwidth.  A CTA pair
// shares its operands through the pair MMA: each CTA loads only ITS 128 rows of A and ITS half of the BN rows of B per
// k-block and the tensor cores of both SMs read both halves of B, which gives 128 FLOP per loaded byte at BN = 256.  At
// BN = 128 (layers with 128 output channels) the loaded bytes per FLOP equal those of a 256 x 128 single-CTA tile, but
// each SM reads 6 KB instead of 8 KB of shared memory per 128 x 128 x 16 step, which is what bounds that tile.
//
// Layout of the work (per cluster; both CTAs run the same warp roles):
//   warp 0      TMA producer: own A half and own B half of every k-block; the byte counts of BOTH CTAs are signalled on
//               the leader's "full" barrier (tensor-map copies with .cta_group::2; every load is a unicast copy into
//               the issuing CTA's own shared memory)
//   warp 1      leader CTA only: tcgen05.mma.cta_group::2 issuer; tcgen05.commit with a CTA mask of 0b11 releases the
//               stage in both CTAs and publishes the finished accumulator to both epilogues
//   warps 2..9  epilogue of the CTA's own 128 rows x 256 columns (TMEM -> registers -> fused math -> TMA store); the
//               epilogue warps of both CTAs arrive on the leader's "accumulator free" barrier
// Every wait is bounded; a CTA that gives up raises the library's error word and still reaches the two cluster barriers
// that frame the kernel, so its peer is never left waiting on hardware.
#pragma once
#include <cstdlib>

#include "gemm_tn.cuh"

namespace pnm {

// Two staging buffers per epilogue warp in every mode: a third buffer for the auxiliary operand costs a stage and
// measured slower on K = 3072 (132 vs 124 us) and no faster on K = 768.
template <int BN, int MODE>
struct PairCfg {
  static constexpr int NBUF = 2;
  static constexpr int B_ROWS = BN / 2;                             // rows of B (output columns) this CTA loads
  static constexpr int STAGE_BYTES = kBM * kBK * 2 + B_ROWS * kBK * 2;
  static constexpr int STAGING = 8 * NBUF * kChunkBytes;           // 8 epilogue warps x NBUF buffers x 4 KB
  static constexpr int BUDGET = 232448 - 1024 - 512;
  static constexpr int STAGES_RAW = (BUDGET - STAGING) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + STAGING + 512;
  static constexpr int TMEM_COLS = 2 * BN;                         // two accumulators
  static_assert(BN == 128 || BN == 256, "pair tile is 256 x 128 or 256 x 256");
  static_assert(STAGES >= 4 && SMEM <= 232448, "paired GEMM: shared memory budget");
};

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory location in the CTA of rank `rank` of this cluster (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load into THIS CTA's shared memory whose bytes are counted on a barrier of the pair's leader CTA.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(void* smem_dst, const CUtensorMap* m, uint32_t leader_bar, int c, int x, int y, int n) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(leader_bar), "r"(c), "r"(x), "r"(y), "r"(n)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' 128 rows] * B[both CTAs' column halves]
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in BOTH CTAs once the pair MMAs issued so far have retired.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

// The kernel reads GemmArgs with num_m_tiles counting 256-row PAIR tiles; in convolution mode M is the number of valid
// 128-pixel tiles x 128 (the last pair may own a single tile) and halo is 0.
template <int BN, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2 /* halo: 7-row box */,
                    const __grid_constant__ CUtensorMap tmA3 /* halo: upper neighbour's row */,
                    const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
                    const __grid_constant__ CUtensorMap tmX /* Z (store), aux (load) or, halo: lower neighbour's row */,
                    const GemmArgs g) {
  using Cfg = PairCfg<BN, MODE>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NBUF = Cfg::NBUF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = base + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::STAGING);
  uint64_t* full = bars;                              // leader's copies are the live ones
  uint64_t* empty = bars + STAGES;                    // per CTA, released by the leader's commits
  uint64_t* tfull = bars + 2 * STAGES;                // per CTA, published by the leader's commits
  uint64_t* tempty = tfull + 2;                       // leader's copies are the live ones (16 arrivals)
  uint64_t* auxbar = tempty + 2;                      // [8 warps][NBUF], per CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(auxbar + 8 * NBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = g.num_m_tiles * g.num_n_tiles;
  const int num_kb = (g.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 16); }
    for (int i = 0; i < 8 * NBUF; ++i) mbar_init(&auxbar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmC);
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                 // both CTAs' barriers exist before any remote arrival or copy
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool up_ready = false, down_ready = false;
      for (int tile = cluster_id; tile < num_tiles; tile += num_clusters) {
        const int mt = tile / g.num_n_tiles, nt = tile % g.num_n_tiles;
        const int mt1 = 2 * mt + int(rank);                       // own 128-row tile of A
        const int col0 = nt * BN + int(rank) * Cfg::B_ROWS;       // own rows of B (output columns)
        int cn = 0, cy0 = 0, cx0 = 0;
        if (g.conv) conv_tile_origin(g, mt1, cn, cy0, cx0);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = base + s * Cfg::STAGE_BYTES;
          if (leader) mbar_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
          const uint32_t lbar = map_to_cta(smem_u32(&full[s]), 0);
          const int k = kb * kBK;
          if (g.conv) {
            const int tap = k / g.cin, c0 = k - tap * g.cin;
            const int xs = cx0 + tap % g.ksize - g.pad, ys = cy0 + tap / g.ksize - g.pad;
            if (g.halo && ys < 0 && g.has_up) {
              // box rows -1 .. 6: row -1 is the upper neighbour's published bottom row (peer memory, plain copy), rows 0 .. 6 local
              if (!up_ready) {
                if (!wait_remote_flag(g.flag_up, g.halo_epoch, abort_flag, g.err, g.halo_budget_ns)) { ok = false; break; }
                up_ready = true;
              }
              tma_load_4d_pair(sa, &tmA3, lbar, c0, xs, 0, cn);
              tma_load_4d_pair(sa + kConvTileW * 128, &tmA2, lbar, c0, xs, 0, cn);
            } else if (g.halo && ys + kConvTileH > g.img_h && g.has_down) {
              // box rows H-7 .. H: rows H-7 .. H-1 local, row H is the lower neighbour's published top row
              if (!down_ready) {
                if (!wait_remote_flag(g.flag_down, g.halo_epoch, abort_flag, g.err, g.halo_budget_ns)) { ok = false; break; }
                down_ready = true;
              }
              tma_load_4d_pair(sa, &tmA2, lbar, c0, xs, ys, cn);
              tma_load_4d_pair(sa + (kConvTileH - 1) * kConvTileW * 128, &tmX, lbar, c0, xs, 0, cn);
            } else {
              tma_load_4d_pair(sa, &tmA, lbar, c0, xs, ys, cn);
            }
          } else {
            tma_load_2d_pair(sa, &tmA, lbar, k, mt1 * kBM);
          }
          tma_load_2d_pair(sa + kBM * kBK * 2, &tmB, lbar, k, col0);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader CTA)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, BN, false, false);
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++tc) {
        const int acc = tc & 1;
        const uint32_t aph = (tc >> 1) & 1;
        if (!mbar_wait(&tempty[acc], aph ^ 1, abort_flag, g.err, ERR_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, g.err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          uint8_t* sa = base + s * Cfg::STAGE_BYTES;
          const uint64_t ad = make_smem_desc(smem_u32(sa), 16, 1024, 2);
          const uint64_t bd = make_smem_desc(smem_u32(sa + kBM * kBK * 2), 16, 1024, 2);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_f16_pair(d, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(&empty[s]);
        }
        if (ok) umma_commit_pair(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int e = warp - 2, q = warp & 3, h = e >> 2;
    constexpr int CH = BN / 128;                       // 64-column chunks per warp per tile (half of the BN columns)
    uint8_t* stg = staging + e * NBUF * kChunkBytes;
    uint64_t* mybar = auxbar + e * NBUF;
    const uint32_t tempty_leader[2] = {map_to_cta(smem_u32(&tempty[0]), 0), map_to_cta(smem_u32(&tempty[1]), 0)};
    uint32_t use = 0, tc = 0;
    bool ok = true;

    auto item_coords = [&](uint32_t item, int& r0, int& c0) -> bool {
      const int tile = cluster_id + int(item / CH) * num_clusters;
      if (tile >= num_tiles) return false;
      const int mt = tile / g.num_n_tiles, nt = tile % g.num_n_tiles;
      r0 = (2 * mt + int(rank)) * kBM + q * 32;
      c0 = nt * BN + h * (BN / 2) + int(item % CH) * 64;
      return true;
    };
    auto issue_aux = [&](uint32_t item) {
      int r0, c0;
      if (!item_coords(item, r0, c0)) return;
      if (lane == 0) {
        tma_store_wait_read<NBUF - 2>();               // the buffer's previous result has left
        const int b = item % NBUF;
        mbar_expect_tx(&mybar[b], kChunkBytes);
        tma_load_2d(stg + b * kChunkBytes, &tmX, &mybar[b], c0, r0);
      }
    };
    if (MODE == MODE_AUX) issue_aux(0);

    uint32_t item = 0;
    for (int tile = cluster_id; ok && tile < num_tiles; tile += num_clusters, ++tc) {
      const int acc = tc & 1;
      const uint32_t aph = (tc >> 1) & 1;
      if (!mbar_wait(&tfull[acc], aph, abort_flag, g.err, ERR_WAIT_TMEM_FULL)) break;
      tc_fence_after();
#pragma unroll 1
      for (int ci = 0; ci < CH; ++ci, ++item) {
        int r0, c0;
        item_coords(item, r0, c0);
        if (MODE == MODE_AUX) issue_aux(item + 1);
        float v[64];
        const uint32_t taddr = tmem_base + acc * BN + h * (BN / 2) + ci * 64 + (uint32_t(q * 32) << 16);
        tmem_ld32(taddr, v);
        tmem_ld32(taddr + 32, v + 32);
        tmem_ld_wait();
        if (ci == CH - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty_leader[acc]);
        }
        const bool store_ok = (r0 < g.M) && (c0 < g.N);
        if (g.bias) {
          if (c0 + 64 <= g.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float4 b = __ldg(reinterpret_cast<const float4*>(g.bias + c0) + j);
              v[4 * j] += b.x; v[4 * j + 1] += b.y; v[4 * j + 2] += b.z; v[4 * j + 3] += b.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) if (c0 + j < g.N) v[j] += __ldg(g.bias + c0 + j);
          }
        }
        if (MODE == MODE_Z) {                          // second output: the pre-activation
          const int b = use % NBUF;
          if (lane == 0) tma_store_wait_read<NBUF - 1>();
          __syncwarp();
          stage_write_row(stg + b * kChunkBytes, lane, v);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (store_ok) tma_store_2d(stg + b * kChunkBytes, &tmX, c0, r0);
            tma_store_commit();
          }
          ++use;
        }
        switch (g.act) {
          case ACT_GELU:
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = gelu_f(v[j]);
            break;
          case ACT_SILU:
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = silu_f(v[j]);
            break;
          case ACT_RELU:
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = fmaxf(v[j], 0.f);
            break;
          default: break;
        }
        int b = use % NBUF;
        if (MODE == MODE_AUX) {
          b = item % NBUF;
          const uint32_t bph = (item / NBUF) & 1;
          if (!mbar_wait(&mybar[b], bph, abort_flag, g.err, ERR_WAIT_AUX)) { ok = false; break; }
          float a[64];
          stage_read_row(stg + b * kChunkBytes, lane, a);
          switch (g.aux_mode) {
            case AUX_ADD:
#pragma unroll
              for (int j = 0; j < 64; ++j) v[j] += a[j];
              break;
            case AUX_DGELU:
#pragma unroll
              for (int j = 0; j < 64; ++j) v[j] *= gelu_grad_f(a[j]);
              break;
            case AUX_DSILU:
#pragma unroll
              for (int j = 0; j < 64; ++j) v[j] *= silu_grad_f(a[j]);
              break;
            case AUX_DRELU:
#pragma unroll
              for (int j = 0; j < 64; ++j) v[j] = a[j] > 0.f ? v[j] : 0.f;
              break;
            default: break;
          }
        } else {
          if (lane == 0) tma_store_wait_read<NBUF - 1>();
          __syncwarp();
        }
        stage_write_row(stg + b * kChunkBytes, lane, v);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (g.conv) {
            // this warp's 32 rows are two image rows of 16 pixels: one 4-D box; the copy engine clips at the image edge
            int n, y0, x0;
            conv_tile_origin(g, r0 / kBM, n, y0, x0);
            const int yy = y0 + 2 * q;
            if (store_ok && yy < g.img_h) tma_store_4d(stg + b * kChunkBytes, &tmC, c0, x0, yy, n);
          } else if (store_ok) tma_store_2d(stg + b * kChunkBytes, &tmC, c0, r0);
          tma_store_commit();
        }
        ++use;
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }
  // ------------------------------------------------------------- teardown
  if (*abort_flag) {
    // a wait ran out: copies of this pair may still be in flight towards this CTA's shared memory; give them time to land
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {}
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // the peer has issued its last read of this CTA's operands
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------- host
inline int pair_gemm_min_k() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("PNM_GEMM_PAIR_MIN_K");         // tuning knob; the default is where the pair tile starts to win
    v = e ? atoi(e) : 512;
    if (v < 64) v = 64;
  }
  return v;
}

// Shapes the pair kernel takes over from the single-CTA one: one A source, no column scale, no softmax epilogues, no
// stacked batch, and enough work per dimension for 256-row tiles to pay.  The halo-fused 3 x 3 convolution of a row-sharded
// image is carried too (boundary rows from the neighbours' published buffers after a bounded wait on their flags).
inline bool pair_gemm_applicable(const GemmCall& c) {
  if (c.batch > 1 || c.split_m || c.scale || c.group_out || c.max_ctas) return false;
  if (c.halo && (!c.conv || c.ksize != 3 || (c.img_h % kConvTileH))) return false;
  if (c.K1 != c.K || c.K2 != c.K) return false;
  if (c.act == ACT_SOFTMAX64 || c.aux_mode == AUX_DSOFTMAX) return false;
  if (c.Z && c.AUX) return false;
  if (c.conv) {
    // 3 x 3 (and wider) windows over >= 64 channels: K >= 576.  Layers of 65 .. 128 output channels take the 256 x 128
    // pair tile, wider ones the 256 x 256 tile.
    return !c.Z && !c.AUX && c.N > 64 && c.K >= pair_gemm_min_k() && (long long)c.img_n * c.img_h * c.img_w >= 8192;
  }
  if (c.N < 256 || c.M < 2048) return false;
  if (c.K >= pair_gemm_min_k()) return true;
  // two outputs of >= 1024 columns: the wider tile also pays at K = 256 (measured 1.00 vs 1.05 ms at 1 M rows); plain and
  // auxiliary-operand GEMMs of that depth are faster on the single-CTA kernel (0.19 vs 0.23 ms, 0.26 vs 0.32 ms)
  return c.Z != nullptr && c.K >= 256 && c.N >= 1024;
}

template <int BN, int MODE>
inline int launch_gemm_tn_pair(const GemmCall& c, int num_sms, int* err_word, cudaStream_t stream) {
  using Cfg = PairCfg<BN, MODE>;
  CUtensorMap tA, tA2, tA3, tB, tC, tX;
  GemmArgs g = {};
  g.M = c.M; g.N = c.N; g.K = c.K; g.K1 = c.K; g.K2 = c.K;
  g.bias = c.bias; g.act = c.act; g.aux_mode = c.aux_mode;
  g.err = err_word;
  int tiles128 = (c.M + kBM - 1) / kBM;
  if (c.conv) {
    if (MODE != MODE_PLAIN) return -19;
    if (make_tmap_nhwc_b16(&tA, c.A, c.img_n, c.img_h, c.img_w, c.cin, kConvTileH, kConvTileW)) return -10;
    if (make_tmap_nhwc_b16(&tC, c.C, c.img_n, c.img_h, c.img_w, c.N, 2, kConvTileW)) return -13;
    g.conv = 1; g.cin = c.cin; g.ksize = c.ksize; g.pad = c.ksize / 2; g.img_h = c.img_h; g.img_n = c.img_n;
    g.tiles_x = (c.img_w + kConvTileW - 1) / kConvTileW;
    g.tiles_y = (c.img_h + kConvTileH - 1) / kConvTileH;
    tiles128 = c.img_n * g.tiles_x * g.tiles_y;
    g.M = tiles128 * kBM;                  // every row of a valid tile is "in range"; the copy engine clips at image edges
    tA2 = tA; tA3 = tA;
    if (c.halo) {
      if (make_tmap_nhwc_b16(&tA2, c.A, c.img_n, c.img_h, c.img_w, c.cin, kConvTileH - 1, kConvTileW)) return -11;
      if (c.up_rows && make_tmap_nhwc_b16(&tA3, c.up_rows, c.img_n, 1, c.img_w, c.cin, 1, kConvTileW)) return -18;
      g.halo = 1; g.has_up = c.up_rows != nullptr; g.has_down = c.down_rows != nullptr;
      g.flag_up = c.flag_up; g.flag_down = c.flag_down; g.halo_epoch = c.halo_epoch;
      g.halo_budget_ns = c.halo_budget_s > 0.0 ? (unsigned long long)(c.halo_budget_s * 1e9) : kWaitBudgetNs;
    }
  } else {
    if (make_tmap_2d_b16(&tA, c.A, c.M, c.K, c.lda, kBM, kBK)) return -10;
    if (make_tmap_2d_b16(&tC, c.C, c.M, c.N, c.ldc, 32, 64)) return -13;
  }
  if (make_tmap_2d_b16(&tB, c.B, c.N, c.K, c.ldb, Cfg::B_ROWS, kBK)) return -12;
  if (MODE == MODE_Z) { if (make_tmap_2d_b16(&tX, c.Z, c.M, c.N, c.ldz, 32, 64)) return -14; }
  else if (MODE == MODE_AUX) { if (make_tmap_2d_b16(&tX, c.AUX, c.M, c.N, c.ldaux, 32, 64)) return -15; }
  else if (c.conv && c.halo && c.down_rows) { if (make_tmap_nhwc_b16(&tX, c.down_rows, c.img_n, 1, c.img_w, c.cin, 1, kConvTileW)) return -15; }
  else tX = tC;
  if (!c.conv) { tA2 = tA; tA3 = tA; }
  g.num_m_tiles = (tiles128 + 1) / 2;
  g.num_n_tiles = (c.N + BN - 1) / BN;
  static unsigned long long attr_mask = 0;
  if (first_use_on_device(attr_mask)) {
    if (cudaFuncSetAttribute(gemm_tn_pair_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
      return -16;
  }
  const int tiles = g.num_m_tiles * g.num_n_tiles;
  int clusters = num_sms / 2;
  if (clusters > tiles) clusters = tiles;
  if (clusters < 1) return -17;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_tn_pair_kernel<BN, MODE>, tA, tA2, tA3, tB, tC, tX, g) != cudaSuccess) return -3;
  return 0;
}

}  // namespace pnm
