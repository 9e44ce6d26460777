// Out[Na,Nb] (fp32) += A[M,Na]^T * B[M,Nb], optionally colsum[Na] += sum_m A[m,:].
//
// This is the weight-gradient / token-reduction shape: the reduction runs over the huge
// row dimension M, the output is small.  Both operands are read exactly as they sit in
// memory (row-major, rows = reduction index), i.e. as MN-major tcgen05 operands: TMA
// brings 64-row x 64-column boxes (128-byte swizzle) and the shared-memory descriptors
// use SBO = 1024 (eight reduction rows) and LBO = box size (next 64 columns).
// Grid = (output tiles) x (splits of M); each CTA accumulates its slice in TMEM and adds
// the tile to the fp32 output with vector reductions (red.global.add).  The column sum
// is one extra N=16 MMA per step against a shared tile filled with ones, so the bias
// gradient / slice norm costs no extra pass over A.
//
// Convolution weight gradient (conv != 0): dW[co, tap, ci] = sum over output pixels p of dY[p, co] * X[p + tap, ci] is the
// same reduction with the pixels as the reduction index.  A reduction block is a 4 x 16 patch of pixels: A (dY) and
// B (X shifted by the tap of the output column block) both arrive as 4-D TMA boxes of an NHWC tensor, whose shared
// memory layout (64 rows of 128 bytes) is that of the 2-D boxes above; coordinates outside the image read as zeros,
// which is the padding.  For a height slab of a row-sharded image (halo != 0) the input row just above / below the slab
// comes from the neighbour's published boundary row (peer-mapped, plain TMA load) after a bounded wait on its flag.
#pragma once
#include "common.cuh"
#include "tmap.cuh"
#include "pnm_internal.h"
#include "gemm_tn.cuh"

namespace pnm {

constexpr int kNtThreads = 192;  // warp0 producer, warp1 MMA, warps 2..5 epilogue
constexpr int kNtBK = 64;        // reduction rows per stage

template <int BNB>
struct NtCfg {
  static constexpr int A_BYTES = 2 * 64 * kNtBK * 2;          // 128 output rows = 2 boxes of 64 columns
  static constexpr int B_BYTES = (BNB / 64) * 64 * kNtBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BNB == 256) ? 4 : 6;
  static constexpr int ONES_BYTES = 2048;
  static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + ONES_BYTES + 256;
  static constexpr int TMEM_COLS = 512;
};

struct NtArgs {
  int M, Na, Nb;
  int rows_per_split;  // multiple of 64
  int tiles_a, tiles_b;
  float* out; int ldo;
  float* colsum;       // [Na] or null
  int* err;
  // stacked batch (batch > 1): `batch` problems of batch_rows reduction rows one after the other in A and B; problem b adds
  // into out + b * out_stride and colsum + b * Na.  Grid = tiles x splits x batch.
  int batch, batch_rows, splits;
  long long out_stride;
  // convolution weight gradient
  int conv, img_n, img_h, img_w, cin, tiles_x, tiles_y;
  int halo, has_up, has_down;
  const uint32_t* flag_up;
  const uint32_t* flag_down;
  uint32_t halo_epoch;
  unsigned long long halo_budget_ns;
};

constexpr int kWgTileH = 4;
constexpr int kWgTileW = 16;

template <int BNB>
__global__ void __launch_bounds__(kNtThreads, 1)
gemm_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmB3 /* conv + halo: 3-row box of X */,
               const __grid_constant__ CUtensorMap tmUp, const __grid_constant__ CUtensorMap tmDown, const NtArgs g) {
  using Cfg = NtCfg<BNB>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ones = base + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ones + Cfg::ONES_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x % (g.tiles_a * g.tiles_b);
  const int split_all = blockIdx.x / (g.tiles_a * g.tiles_b);
  const int prob = g.batch > 1 ? split_all / g.splits : 0;
  const int split = g.batch > 1 ? split_all % g.splits : split_all;
  const int ta = tile / g.tiles_b, tb = tile % g.tiles_b;
  const int m_lo = prob * g.batch_rows, m_hi = g.batch > 1 ? m_lo + g.batch_rows : g.M;
  const int m_begin = m_lo + split * g.rows_per_split;
  int m_end = m_begin + g.rows_per_split;
  if (m_end > m_hi) m_end = m_hi;
  const int num_kb = m_end > m_begin ? (m_end - m_begin + kNtBK - 1) / kNtBK : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(tfull, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  // ones tile (bf16 1.0 = 0x3f80)
  for (int i = threadIdx.x; i < Cfg::ONES_BYTES / 4; i += kNtThreads) reinterpret_cast<uint32_t*>(ones)[i] = 0x3f803f80u;
  fence_async_smem();
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
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
        if (g.conv) {
          const int patch = m / kNtBK;
          const int per_img = g.tiles_x * g.tiles_y;
          const int n = patch / per_img, r = patch - n * per_img;
          const int y0 = (r / g.tiles_x) * kWgTileH, x0 = (r % g.tiles_x) * kWgTileW;
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
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
#pragma unroll
          for (int i = 0; i < 2; ++i) tma_load_4d(sa + i * 8192, &tmA, &full[s], ta * 128 + i * 64, x0, y0, n);
#pragma unroll
          for (int i = 0; i < BNB / 64; ++i) {
            const int col = tb * BNB + i * 64;
            int tap = col / g.cin, c0 = col - tap * g.cin;
            if (tap >= 9) { tap = 4; c0 = g.cin; }           // past the last tap: channel coordinate out of range reads zeros
            const int xs = x0 + tap % 3 - 1, ys = y0 + tap / 3 - 1;
            uint8_t* dst = sb + i * 8192;
            if (g.halo && ys < 0 && g.has_up) {
              tma_load_4d(dst, &tmUp, &full[s], c0, xs, 0, n);                          // row -1: upper neighbour's last row
              tma_load_4d(dst + kWgTileW * 128, &tmB3, &full[s], c0, xs, 0, n);         // rows 0 .. 2
            } else if (g.halo && ys + kWgTileH > g.img_h && g.has_down) {
              tma_load_4d(dst, &tmB3, &full[s], c0, xs, ys, n);                         // rows H-3 .. H-1
              tma_load_4d(dst + (kWgTileH - 1) * kWgTileW * 128, &tmDown, &full[s], c0, xs, 0, n);  // row H
            } else {
              tma_load_4d(dst, &tmB, &full[s], c0, xs, ys, n);
            }
          }
        } else {
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
#pragma unroll
          for (int i = 0; i < 2; ++i) tma_load_2d(sa + i * 8192, &tmA, &full[s], ta * 128 + i * 64, m);
#pragma unroll
          for (int i = 0; i < BNB / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, &full[s], tb * BNB + i * 64, m);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, BNB, true, true);
      constexpr uint32_t idesc1 = make_idesc_bf16(128, 16, true, false);
      // ones tile as a K-major, unswizzled operand: every element it can address is 1.0
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
          // 16 reduction rows = 2048 bytes = 128 sixteen-byte units
          umma_f16(tmem_base, ad + 128 * k, bd + 128 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          if (g.colsum) umma_f16(tmem_base + BNB, ad + 128 * k, od, idesc1, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(tfull);
    }
  } else if (num_kb > 0) {
    const int q = warp & 3;
    if (mbar_wait(tfull, 0, abort_flag, g.err, ERR_WAIT_TMEM_FULL)) {
      tc_fence_after();
      const int row = ta * 128 + q * 32 + lane;  // output row (column of A)
      for (int c = 0; c < BNB; c += 32) {
        float v[32];
        tmem_ld32(tmem_base + c + (uint32_t(q * 32) << 16), v);
        tmem_ld_wait();
        const int col0 = tb * BNB + c;
        if (row < g.Na) {
          float* dst = g.out + prob * g.out_stride + size_t(row) * g.ldo + col0;
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
        if (row < g.Na) atomicAdd(g.colsum + prob * g.Na + row, v[0]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

struct NtCall {
  const void* A; int lda;
  const void* B; int ldb;
  float* out; int ldo;
  float* colsum;
  int M, Na, Nb;
  int max_ctas;
  int batch = 1; long long out_stride = 0;   // stacked problems: M is the total row count (M / batch % 64 == 0)
  // convolution weight gradient: A = dY [img_n, img_h, img_w, Na], B = X [img_n, img_h, img_w, cin]; Nb = 9 * cin
  int conv = 0, img_n = 0, img_h = 0, img_w = 0, cin = 0;
  int halo = 0;
  const void* up_rows = nullptr; const void* down_rows = nullptr;
  const uint32_t* flag_up = nullptr; const uint32_t* flag_down = nullptr;
  uint32_t halo_epoch = 0;
  double halo_budget_s = 0.0;
};

template <int BNB>
inline int launch_gemm_nt(const NtCall& c, int num_sms, int* err_word, cudaStream_t stream) {
  using Cfg = NtCfg<BNB>;
  CUtensorMap tA, tB, tB3, tUp, tDown;
  NtArgs g;
  g.conv = c.conv; g.img_n = c.img_n; g.img_h = c.img_h; g.img_w = c.img_w; g.cin = c.cin;
  g.tiles_x = g.tiles_y = 0;
  g.halo = c.conv ? c.halo : 0; g.has_up = c.up_rows != nullptr; g.has_down = c.down_rows != nullptr;
  g.flag_up = c.flag_up; g.flag_down = c.flag_down; g.halo_epoch = c.halo_epoch;
  g.halo_budget_ns = c.halo_budget_s > 0.0 ? (unsigned long long)(c.halo_budget_s * 1e9) : kWaitBudgetNs;
  int M = c.M;
  if (c.conv) {
    if (c.cin % 64 || c.Nb != 9 * c.cin || c.Na < 64) return -24;
    if (g.halo && (c.img_h % kWgTileH)) return -24;
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
  g.tiles_a = (c.Na + 127) / 128;
  g.tiles_b = (c.Nb + BNB - 1) / BNB;
  const int tiles = g.tiles_a * g.tiles_b;
  const int nprob = c.batch > 1 ? c.batch : 1;
  if (nprob > 1 && (c.conv || M % (nprob * kNtBK))) return -25;
  const int cap = c.max_ctas > 0 ? c.max_ctas : num_sms;
  int splits = cap / (tiles * nprob);
  if (splits < 1) splits = 1;
  const int kblocks = (M / nprob + kNtBK - 1) / kNtBK;
  if (splits > kblocks) splits = kblocks;
  int per = (kblocks + splits - 1) / splits;
  g.rows_per_split = per * kNtBK;
  splits = (kblocks + per - 1) / per;
  g.out = c.out; g.ldo = c.ldo; g.colsum = c.colsum; g.err = err_word;
  g.batch = nprob; g.batch_rows = M / nprob; g.splits = splits; g.out_stride = c.out_stride;
  static unsigned long long attr_mask = 0;
  if (first_use_on_device(attr_mask)) {
    if (cudaFuncSetAttribute(gemm_nt_kernel<BNB>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
      return -22;
  }
  gemm_nt_kernel<BNB><<<tiles * splits * nprob, kNtThreads, Cfg::SMEM, stream>>>(tA, tB, tB3, tUp, tDown, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -23;
}

}  // namespace pnm
