// Out[Na,Nb] (fp32) += A[M,Na]^T * B[M,Nb] (+ column sums of A) on CTA PAIRS: the reduction GEMM of gemm_nt.cuh with one
// 256 x BNB output tile per cluster of two CTAs (tcgen05.mma.cta_group::2).  CTA r of the pair loads the 128 columns of
// A that become ITS 128 output rows and half of the BNB columns of B per 64 reduction rows (32 KB instead of the 48 KB a
// single CTA loads for half as many products); the leader CTA issues the MMAs for both SMs; each CTA adds its 128 output
// rows to the fp32 result with vector reductions.  Same operand layout as the single-CTA kernel (MN-major boxes of 64
// columns, 128-byte swizzle), same convolution weight-gradient mode (4 x 16 pixel patches as reduction blocks, shifted
// 4-D boxes of the input) including the halo variant of a row-sharded image (boundary rows from the neighbours'
// published buffers after a bounded wait on their flags).  Used when the output has at least 256 rows.
#pragma once
#include "gemm_nt.cuh"
#include "gemm_tn_pair.cuh"

namespace pnm {

template <int BNB>
struct NtPairCfg {
  static constexpr int A_BYTES = 2 * 64 * kNtBK * 2;                 // own 128 output rows = 2 boxes of 64 columns
  static constexpr int B_BOXES = BNB / 128;                          // own half of the BNB columns, in boxes of 64
  static constexpr int B_BYTES = B_BOXES * 64 * kNtBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int ONES_BYTES = 2048;
  static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + ONES_BYTES + 256;
  static constexpr int TMEM_COLS = 512;
  static_assert(BNB == 128 || BNB == 256, "pair tile is 256 x 128 or 256 x 256");
  static_assert(SMEM <= 232448, "paired reduction GEMM: shared memory budget");
};

template <int BNB>
__global__ void __launch_bounds__(kNtThreads, 1)
gemm_nt_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmB3 /* conv + halo: 3-row box of X */,
                    const __grid_constant__ CUtensorMap tmUp, const __grid_constant__ CUtensorMap tmDown, const NtArgs g) {
  using Cfg = NtPairCfg<BNB>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ones = base + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ones + Cfg::ONES_BYTES);
  uint64_t* full = bars;                     // leader's copies are the live ones
  uint64_t* empty = bars + STAGES;           // per CTA, released by the leader's commits
  uint64_t* tfull = bars + 2 * STAGES;       // per CTA, published by the leader's commit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int tile = cluster_id % (g.tiles_a * g.tiles_b);
  const int split = cluster_id / (g.tiles_a * g.tiles_b);
  const int ta = tile / g.tiles_b, tb = tile % g.tiles_b;     // tiles_a counts 256-row pair tiles
  const int m_begin = split * g.rows_per_split;
  int m_end = m_begin + g.rows_per_split;
  if (m_end > g.M) m_end = g.M;
  const int num_kb = m_end > m_begin ? (m_end - m_begin + kNtBK - 1) / kNtBK : 0;
  const int a_col0 = ta * 256 + int(rank) * 128;              // own columns of A = own output rows
  const int b_col0 = tb * BNB + int(rank) * (BNB / 2);        // own columns of B

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(tfull, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < Cfg::ONES_BYTES / 4; i += kNtThreads) reinterpret_cast<uint32_t*>(ones)[i] = 0x3f803f80u;
  fence_async_smem();
  if (warp == 1) { tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                        // both CTAs' barriers and ones tiles exist before any remote arrival or MMA
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bool up_ready = false, down_ready = false;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, g.err, ERR_WAIT_EMPTY)) break;
        uint8_t* sa = base + s * Cfg::STAGE_BYTES;
        uint8_t* sb = sa + Cfg::A_BYTES;
        const int m = m_begin + kb * kNtBK;
        int n = 0, y0 = 0, x0 = 0;
        if (g.conv) {
          const int patch = m / kNtBK;
          const int per_img = g.tiles_x * g.tiles_y;
          n = patch / per_img;
          const int r = patch - n * per_img;
          y0 = (r / g.tiles_x) * kWgTileH; x0 = (r % g.tiles_x) * kWgTileW;
          // the flags are looked at before the stage is armed, so that a time-out leaves no barrier half expected
          bool flags_ok = true;
          if (g.halo) {
            if (y0 == 0 && g.has_up && g.flag_up && !up_ready) {
              flags_ok = wait_remote_flag(g.flag_up, g.halo_epoch, abort_flag, g.err, g.halo_budget_ns);
              up_ready = flags_ok;
            }
            if (flags_ok && y0 + kWgTileH >= g.img_h && g.has_down && g.flag_down && !down_ready) {
              flags_ok = wait_remote_flag(g.flag_down, g.halo_epoch, abort_flag, g.err, g.halo_budget_ns);
              down_ready = flags_ok;
            }
          }
          if (!flags_ok) break;
        }
        if (leader) mbar_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
        const uint32_t lbar = map_to_cta(smem_u32(&full[s]), 0);
        if (g.conv) {
#pragma unroll
          for (int i = 0; i < 2; ++i) tma_load_4d_pair(sa + i * 8192, &tmA, lbar, a_col0 + i * 64, x0, y0, n);
#pragma unroll
          for (int i = 0; i < Cfg::B_BOXES; ++i) {
            const int col = b_col0 + i * 64;
            int tap = col / g.cin, c0 = col - tap * g.cin;
            if (tap >= 9) { tap = 4; c0 = g.cin; }           // past the last tap: channel coordinate out of range reads zeros
            const int xs = x0 + tap % 3 - 1, ys = y0 + tap / 3 - 1;
            uint8_t* dst = sb + i * 8192;
            if (g.halo && ys < 0 && g.has_up) {
              tma_load_4d_pair(dst, &tmUp, lbar, c0, xs, 0, n);                          // row -1: upper neighbour's last row
              tma_load_4d_pair(dst + kWgTileW * 128, &tmB3, lbar, c0, xs, 0, n);         // rows 0 .. 2
            } else if (g.halo && ys + kWgTileH > g.img_h && g.has_down) {
              tma_load_4d_pair(dst, &tmB3, lbar, c0, xs, ys, n);                         // rows H-3 .. H-1
              tma_load_4d_pair(dst + (kWgTileH - 1) * kWgTileW * 128, &tmDown, lbar, c0, xs, 0, n);  // row H
            } else {
              tma_load_4d_pair(dst, &tmB, lbar, c0, xs, ys, n);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 2; ++i) tma_load_2d_pair(sa + i * 8192, &tmA, lbar, a_col0 + i * 64, m);
#pragma unroll
          for (int i = 0; i < Cfg::B_BOXES; ++i) tma_load_2d_pair(sb + i * 8192, &tmB, lbar, b_col0 + i * 64, m);
        }
      }
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, BNB, true, true);
      constexpr uint32_t idesc1 = make_idesc_bf16(256, 16, true, false);
      // ones tile as a K-major, unswizzled operand: every element it can address is 1.0 (in both CTAs)
      const uint64_t od = make_smem_desc(smem_u32(ones), 128, 256, 0);
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, abort_flag, g.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        uint8_t* sa = base + s * Cfg::STAGE_BYTES;
        const uint64_t ad = make_smem_desc(smem_u32(sa), 8192, 1024, 2);
        const uint64_t bd = make_smem_desc(smem_u32(sa + Cfg::A_BYTES), 8192, 1024, 2);
#pragma unroll
        for (int k = 0; k < kNtBK / 16; ++k) {
          umma_f16_pair(tmem_base, ad + 128 * k, bd + 128 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          if (g.colsum) umma_f16_pair(tmem_base + BNB, ad + 128 * k, od, idesc1, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit_pair(&empty[s]);
      }
      if (ok) umma_commit_pair(tfull);
    }
  } else if (num_kb > 0) {
    const int q = warp & 3;
    if (mbar_wait(tfull, 0, abort_flag, g.err, ERR_WAIT_TMEM_FULL)) {
      tc_fence_after();
      const int row = a_col0 + q * 32 + lane;                 // output row (column of A)
      for (int c = 0; c < BNB; c += 32) {
        float v[32];
        tmem_ld32(tmem_base + c + (uint32_t(q * 32) << 16), v);
        tmem_ld_wait();
        const int col0 = tb * BNB + c;
        if (row < g.Na) {
          float* dst = g.out + size_t(row) * g.ldo + col0;
          if (col0 + 32 <= g.Nb && (g.ldo & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j), "f"(v[4 * j]),
                           "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                           : "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) if (col0 + j < g.Nb) atomicAdd(dst + j, v[j]);
          }
        }
      }
      if (g.colsum && tb == 0) {
        float v[32];
        tmem_ld32(tmem_base + BNB + (uint32_t(q * 32) << 16), v);
        tmem_ld_wait();
        if (row < g.Na) atomicAdd(g.colsum + row, v[0]);
      }
    }
  }
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {}
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                        // the peer has issued its last read of this CTA's operands
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

inline bool pair_gemm_nt_applicable(const NtCall& c) {
  if (c.batch > 1 || c.max_ctas) return false;
  if (c.halo && (!c.conv || (c.img_h % kWgTileH))) return false;
  if (c.Na < 256 || c.Nb < 128) return false;
  const long long rows = c.conv ? (long long)c.img_n * c.img_h * c.img_w : c.M;
  return rows >= 8192;
}

template <int BNB>
inline int launch_gemm_nt_pair(const NtCall& c, int num_sms, int* err_word, cudaStream_t stream) {
  using Cfg = NtPairCfg<BNB>;
  CUtensorMap tA, tB, tB3, tUp, tDown;
  NtArgs g = {};
  g.conv = c.conv; g.img_n = c.img_n; g.img_h = c.img_h; g.img_w = c.img_w; g.cin = c.cin;
  g.halo = c.conv ? c.halo : 0; g.has_up = c.up_rows != nullptr; g.has_down = c.down_rows != nullptr;
  g.flag_up = c.flag_up; g.flag_down = c.flag_down; g.halo_epoch = c.halo_epoch;
  g.halo_budget_ns = c.halo_budget_s > 0.0 ? (unsigned long long)(c.halo_budget_s * 1e9) : kWaitBudgetNs;
  int M = c.M;
  if (c.conv) {
    if (c.cin % 64 || c.Nb != 9 * c.cin || c.Na < 64) return -24;
    if (make_tmap_nhwc_b16(&tA, c.A, c.img_n, c.img_h, c.img_w, c.Na, kWgTileH, kWgTileW)) return -20;
    if (make_tmap_nhwc_b16(&tB, c.B, c.img_n, c.img_h, c.img_w, c.cin, kWgTileH, kWgTileW)) return -21;
    tB3 = tB; tUp = tB; tDown = tB;
    if (g.halo) {
      if (make_tmap_nhwc_b16(&tB3, c.B, c.img_n, c.img_h, c.img_w, c.cin, kWgTileH - 1, kWgTileW)) return -21;
      if (c.up_rows && make_tmap_nhwc_b16(&tUp, c.up_rows, c.img_n, 1, c.img_w, c.cin, 1, kWgTileW)) return -21;
      if (c.down_rows && make_tmap_nhwc_b16(&tDown, c.down_rows, c.img_n, 1, c.img_w, c.cin, 1, kWgTileW)) return -21;
    }
    g.tiles_x = (c.img_w + kWgTileW - 1) / kWgTileW;
    g.tiles_y = (c.img_h + kWgTileH - 1) / kWgTileH;
    M = c.img_n * g.tiles_x * g.tiles_y * kNtBK;       // reduction rows = patches of 64 pixels
  } else {
    if (make_tmap_2d_b16(&tA, c.A, c.M, c.Na, c.lda, kNtBK, 64)) return -20;
    if (make_tmap_2d_b16(&tB, c.B, c.M, c.Nb, c.ldb, kNtBK, 64)) return -21;
    tB3 = tB; tUp = tB; tDown = tB;
  }
  g.M = M; g.Na = c.Na; g.Nb = c.Nb;
  g.tiles_a = (c.Na + 255) / 256;
  g.tiles_b = (c.Nb + BNB - 1) / BNB;
  const int tiles = g.tiles_a * g.tiles_b;
  int splits = (num_sms / 2) / tiles;
  if (splits < 1) splits = 1;
  const int kblocks = (M + kNtBK - 1) / kNtBK;
  if (splits > kblocks) splits = kblocks;
  const int per = (kblocks + splits - 1) / splits;
  g.rows_per_split = per * kNtBK;
  splits = (kblocks + per - 1) / per;
  g.out = c.out; g.ldo = c.ldo; g.colsum = c.colsum; g.err = err_word;
  g.batch = 1; g.batch_rows = M; g.splits = splits; g.out_stride = 0;
  static unsigned long long attr_mask = 0;
  if (first_use_on_device(attr_mask)) {
    if (cudaFuncSetAttribute(gemm_nt_pair_kernel<BNB>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
      return -22;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * tiles * splits);
  cfg.blockDim = dim3(kNtThreads);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemm_nt_pair_kernel<BNB>, tA, tB, tB3, tUp, tDown, g) != cudaSuccess) return -23;
  return 0;
}

}  // namespace pnm
