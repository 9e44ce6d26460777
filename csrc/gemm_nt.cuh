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
#pragma once
#include "common.cuh"
#include "tmap.cuh"

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
};

template <int BNB>
__global__ void __launch_bounds__(kNtThreads, 1)
gemm_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const NtArgs g) {
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
  const int split = blockIdx.x / (g.tiles_a * g.tiles_b);
  const int ta = tile / g.tiles_b, tb = tile % g.tiles_b;
  const int m_begin = split * g.rows_per_split;
  int m_end = m_begin + g.rows_per_split;
  if (m_end > g.M) m_end = g.M;
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
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        const uint32_t ph = (kb / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, g.err, ERR_WAIT_EMPTY)) break;
        uint8_t* sa = base + s * Cfg::STAGE_BYTES;
        uint8_t* sb = sa + Cfg::A_BYTES;
        mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
        const int m = m_begin + kb * kNtBK;
#pragma unroll
        for (int i = 0; i < 2; ++i) tma_load_2d(sa + i * 8192, &tmA, &full[s], ta * 128 + i * 64, m);
#pragma unroll
        for (int i = 0; i < BNB / 64; ++i) tma_load_2d(sb + i * 8192, &tmB, &full[s], tb * BNB + i * 64, m);
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
};

template <int BNB>
inline int launch_gemm_nt(const NtCall& c, int num_sms, int* err_word, cudaStream_t stream) {
  using Cfg = NtCfg<BNB>;
  CUtensorMap tA, tB;
  if (make_tmap_2d_b16(&tA, c.A, c.M, c.Na, c.lda, kNtBK, 64)) return -20;
  if (make_tmap_2d_b16(&tB, c.B, c.M, c.Nb, c.ldb, kNtBK, 64)) return -21;
  NtArgs g;
  g.M = c.M; g.Na = c.Na; g.Nb = c.Nb;
  g.tiles_a = (c.Na + 127) / 128;
  g.tiles_b = (c.Nb + BNB - 1) / BNB;
  const int tiles = g.tiles_a * g.tiles_b;
  const int cap = c.max_ctas > 0 ? c.max_ctas : num_sms;
  int splits = cap / tiles;
  if (splits < 1) splits = 1;
  const int kblocks = (c.M + kNtBK - 1) / kNtBK;
  if (splits > kblocks) splits = kblocks;
  int per = (kblocks + splits - 1) / splits;
  g.rows_per_split = per * kNtBK;
  splits = (kblocks + per - 1) / per;
  g.out = c.out; g.ldo = c.ldo; g.colsum = c.colsum; g.err = err_word;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_nt_kernel<BNB>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
      return -22;
    attr_set = true;
  }
  gemm_nt_kernel<BNB><<<tiles * splits, kNtThreads, Cfg::SMEM, stream>>>(tA, tB, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -23;
}

}  // namespace pnm
