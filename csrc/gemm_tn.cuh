// C[M,N] = epilogue( A[M,K] * B[N,K]^T ), bf16 operands, fp32 accumulation in TMEM.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer (A and B k-blocks of 64 -> 128-byte-swizzled shared tiles)
//   warp 1      tcgen05.mma issuer (one lane), owns the TMEM allocation
//   warps 2..9  epilogue: TMEM -> registers -> fused math -> swizzled staging -> TMA store
// Two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
//
// Fused epilogues (all optional, all applied on fp32 values):
//   x = (acc + bias[col]) * scale[col]            (scale before the activation unless scale_post)
//   Z = x                                         (second output: the pre-activation, MODE_Z)
//   y = act(x)   act in {none, GELU, SiLU, ReLU, softmax over aligned groups of 64 columns}
//   y = y + aux | y * GELU'(aux) | y * SiLU'(aux) | y * ReLU'(aux) | softmax-backward(y; aux = p)
// The auxiliary tile is prefetched by TMA into the same staging buffer the result leaves from.
// A may be split along K into up to three tensors (A | A2 | A3), which gives K-concatenated GEMMs
// without materialising the concatenation.
#pragma once
#include "common.cuh"
#include "tmap.cuh"
#include "pnm_internal.h"

namespace pnm {

enum { ACT_NONE = 0, ACT_GELU = 1, ACT_SILU = 2, ACT_RELU = 3, ACT_SOFTMAX64 = 4 };
enum { AUX_NONE = 0, AUX_ADD = 1, AUX_DGELU = 2, AUX_DSOFTMAX = 3, AUX_DSILU = 4, AUX_DRELU = 5 };
enum { MODE_PLAIN = 0, MODE_Z = 1, MODE_AUX = 2 };

struct GemmArgs {
  int M, N, K, K1, K2;
  const float* bias;
  const float* scale;
  float* group_out;
  int act;
  int aux_mode;
  int scale_post;
  int num_m_tiles, num_n_tiles;
  int* err;
  // stacked batch (batch_m_tiles != 0): A / C hold `batch` problems of batch_m_tiles * 128 rows one after the other, B holds
  // their [N, K] matrices one after the other, bias / scale their [N] vectors: M tile mt belongs to problem mt / batch_m_tiles
  int batch_m_tiles;
  // split_m (BN = 256 instantiation only): a tile is TWO 128-row sub-tiles that share one 128-column B tile, i.e. 256 x 128
  // outputs.  For N <= 128 this reads B once per 256 rows instead of once per 128 (the 128 x 128 tile is bound by the
  // L2 -> shared-memory traffic of its operands); stage size, TMEM layout and the epilogue's warp mapping are those of
  // the 128 x 256 tile with "column half" replaced by "row half".  num_m_tiles counts 256-row tiles.
  int split_m;
  // implicit-GEMM convolution (conv != 0): rows of A are output pixels of an NHWC image, tiled 8 x 16 per M tile;
  // K runs over (tap, input channel); the A tile of k-block (tap, c0) is the input window shifted by the tap
  int conv, tiles_x, tiles_y, cin, ksize, pad, img_h;
  // halo != 0 (3 x 3, img_h % 8 == 0): the image is one horizontal slab of a taller image split over ranks.  The row
  // above / below the slab comes from the neighbour's published boundary row (a peer-mapped buffer read by plain,
  // non-multicast TMA loads) once its flag carries halo_epoch; tiles that need it are scheduled last.
  int halo, has_up, has_down, img_n;
  const uint32_t* flag_up;
  const uint32_t* flag_down;
  uint32_t halo_epoch;
  unsigned long long halo_budget_ns;  // budget of the waits on the neighbours' flags
};

constexpr int kConvTileH = 8;
constexpr int kConvTileW = 16;

__device__ __forceinline__ void conv_tile_origin(const GemmArgs& g, int mt, int& n, int& y0, int& x0) {
  if (g.halo) {
    // interior-first order: tile rows 1 .. tiles_y-2 of every image, then row 0 and row tiles_y-1 (the halo users)
    const int per_row = g.img_n * g.tiles_x;
    const int o = mt / per_row, r = mt - o * per_row;
    n = r / g.tiles_x;
    x0 = (r % g.tiles_x) * kConvTileW;
    const int ty = g.tiles_y <= 2 ? o : (o < g.tiles_y - 2 ? o + 1 : (o == g.tiles_y - 2 ? 0 : g.tiles_y - 1));
    y0 = ty * kConvTileH;
    return;
  }
  const int per_img = g.tiles_x * g.tiles_y;
  n = mt / per_img;
  const int r = mt - n * per_img;
  y0 = (r / g.tiles_x) * kConvTileH;
  x0 = (r % g.tiles_x) * kConvTileW;
}

// Bounded wait (one thread) until a flag written by another GPU reaches `epoch`.
// The rows that the flag announces were written by another GPU with generic-proxy stores and are read here by TMA
// (async proxy): after the acquire succeeds a proxy fence orders the two before the first bulk copy is issued.
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ bool wait_remote_flag(const uint32_t* flag, uint32_t epoch, volatile int* abort_flag, int* err_word,
                                                 unsigned long long budget_ns) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  if (int32_t(v - epoch) >= 0) { fence_proxy_async_global(); return true; }
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (int32_t(v - epoch) >= 0) { fence_proxy_async_global(); return true; }
    if ((++spins & 0xffu) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        atomicCAS(err_word, 0, ERR_WAIT_PEER);
        *abort_flag = 1;
        __threadfence_block();
        return false;
      }
    }
  }
}

constexpr int kGemmThreads = 320;
constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kChunkBytes = 32 * 128;  // 32 rows x 64 bf16

template <int BN, int MODE>
struct GemmCfg {
  static constexpr int NBUF = (MODE == MODE_AUX) ? 3 : 2;
  static constexpr int STAGE_BYTES = kBM * kBK * 2 + BN * kBK * 2;
  static constexpr int STAGING = 8 * NBUF * kChunkBytes;
  static constexpr int BUDGET = 232448 - 1024 /*align*/ - 512 /*barriers*/;
  static constexpr int STAGES_RAW = (BUDGET - STAGING) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int SMEM = 1024 + STAGES * STAGE_BYTES + STAGING + 512;
  static constexpr int TMEM_COLS = 2 * BN;  // 256 or 512: powers of two
  static_assert(STAGES >= 2, "not enough shared memory for a pipeline");
};

__device__ __forceinline__ void stage_write_row(uint8_t* buf, int lane, const float* v) {
  // 64 fp32 -> 64 bf16 = 8 chunks of 16 bytes, chunk j of row r lands at (j ^ (r & 7)).
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 u;
    u.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
    u.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
    u.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
    u.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
    *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = u;
  }
}
__device__ __forceinline__ void stage_read_row(const uint8_t* buf, int lane, float* a) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 u = *reinterpret_cast<const uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4));
    float2 f;
    f = unpack_bf16x2(u.x); a[8 * j + 0] = f.x; a[8 * j + 1] = f.y;
    f = unpack_bf16x2(u.y); a[8 * j + 2] = f.x; a[8 * j + 3] = f.y;
    f = unpack_bf16x2(u.z); a[8 * j + 4] = f.x; a[8 * j + 5] = f.y;
    f = unpack_bf16x2(u.w); a[8 * j + 6] = f.x; a[8 * j + 7] = f.y;
  }
}

template <int BN, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
               const __grid_constant__ CUtensorMap tmA3, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
               const __grid_constant__ CUtensorMap tmX /* Z (store) or aux (load) */, const GemmArgs g) {
  using Cfg = GemmCfg<BN, MODE>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NBUF = Cfg::NBUF;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = base + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::STAGING);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* auxbar = tempty + 2;                      // [8 warps][NBUF]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(auxbar + 8 * 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = g.num_m_tiles * g.num_n_tiles;
  const int num_kb = (g.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 8); }
    for (int i = 0; i < 8 * 3; ++i) mbar_init(&auxbar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmC);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      bool up_ready = false, down_ready = false;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const int mt = tile / g.num_n_tiles, nt = tile % g.num_n_tiles;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, g.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sa = base + s * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + kBM * kBK * 2;
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          const int k = kb * kBK;
          auto load_a = [&](uint8_t* sa, int mt) -> bool {
            if (g.conv) {
              int n, y0, x0;
              conv_tile_origin(g, mt, n, y0, x0);
              const int tap = k / g.cin, c0 = k - tap * g.cin;
              const int xs = x0 + tap % g.ksize - g.pad, ys = y0 + tap / g.ksize - g.pad;
              if (g.halo && ys < 0 && g.has_up) {
                // box rows -1 .. 6: row -1 is the upper neighbour's bottom row, rows 0 .. 6 are local
                if (!up_ready) {
                  if (!wait_remote_flag(g.flag_up, g.halo_epoch, abort_flag, g.err, g.halo_budget_ns)) return false;
                  up_ready = true;
                }
                tma_load_4d(sa, &tmA3, &full[s], c0, xs, 0, n);
                tma_load_4d(sa + kConvTileW * 128, &tmA2, &full[s], c0, xs, 0, n);
              } else if (g.halo && ys + kConvTileH > g.img_h && g.has_down) {
                // box rows H-7 .. H: rows H-7 .. H-1 are local, row H is the lower neighbour's top row
                if (!down_ready) {
                  if (!wait_remote_flag(g.flag_down, g.halo_epoch, abort_flag, g.err, g.halo_budget_ns)) return false;
                  down_ready = true;
                }
                tma_load_4d(sa, &tmA2, &full[s], c0, xs, ys, n);
                tma_load_4d(sa + (kConvTileH - 1) * kConvTileW * 128, &tmX, &full[s], c0, xs, 0, n);
              } else {
                tma_load_4d(sa, &tmA, &full[s], c0, xs, ys, n);
              }
            } else if (k < g.K1) tma_load_2d(sa, &tmA, &full[s], k, mt * kBM);
            else if (k < g.K2) tma_load_2d(sa, &tmA2, &full[s], k - g.K1, mt * kBM);
            else tma_load_2d(sa, &tmA3, &full[s], k - g.K2, mt * kBM);
            return true;
          };
          if (BN == 256 && g.split_m) {
            if (!load_a(sa, 2 * mt) || !load_a(sa + kBM * kBK * 2, 2 * mt + 1)) { ok = false; break; }
            tma_load_2d(sa + 2 * kBM * kBK * 2, &tmB, &full[s], k, nt * 128);
            continue;
          }
          if (!load_a(sa, mt)) { ok = false; break; }
          tma_load_2d(sb, &tmB, &full[s], k, nt * BN + (g.batch_m_tiles ? (mt / g.batch_m_tiles) * g.N : 0));
        }
      }
      if (!ok) {
        // give copies already in flight a bounded chance to land before the CTA leaves
        for (int s = 0; s < STAGES; ++s)
          for (int i = 0; i < (1 << 14) && !mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN, false, false);
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++tc) {
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
          if (BN == 256 && g.split_m) {
            constexpr uint32_t idesc_half = make_idesc_bf16(kBM, 128, false, false);
            const uint64_t ad1 = make_smem_desc(smem_u32(sa + kBM * kBK * 2), 16, 1024, 2);
            const uint64_t bdh = make_smem_desc(smem_u32(sa + 2 * kBM * kBK * 2), 16, 1024, 2);
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
              umma_f16(d, ad + 2 * k, bdh + 2 * k, idesc_half, (kb | k) != 0 ? 1u : 0u);
              umma_f16(d + 128, ad1 + 2 * k, bdh + 2 * k, idesc_half, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty[s]);
            continue;
          }
          const uint64_t bd = make_smem_desc(smem_u32(sa + kBM * kBK * 2), 16, 1024, 2);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_f16(d, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int e = warp - 2, q = warp & 3, h = e >> 2;
    constexpr int CH = BN / 128;  // 64-column chunks per warp per tile
    uint8_t* stg = staging + e * NBUF * kChunkBytes;
    uint64_t* mybar = auxbar + e * 3;
    uint32_t use = 0, tc = 0;
    bool ok = true;

    auto item_coords = [&](uint32_t item, int& r0, int& c0) -> bool {
      const int tile = blockIdx.x + int(item / CH) * gridDim.x;
      if (tile >= num_tiles) return false;
      const int mt = tile / g.num_n_tiles, nt = tile % g.num_n_tiles;
      if (BN == 256 && g.split_m) {             // warp half h owns the rows of sub-tile h, all 128 columns
        r0 = (2 * mt + h) * kBM + q * 32;
        c0 = nt * 128 + int(item % CH) * 64;
        return true;
      }
      r0 = mt * kBM + q * 32;
      c0 = nt * BN + h * (BN / 2) + int(item % CH) * 64;
      return true;
    };
    auto issue_aux = [&](uint32_t item) {
      int r0, c0;
      if (!item_coords(item, r0, c0)) return;
      if (lane == 0) {
        tma_store_wait_read<NBUF - 2 < 0 ? 0 : NBUF - 2>();
        const int b = item % NBUF;
        mbar_expect_tx(&mybar[b], kChunkBytes);
        tma_load_2d(stg + b * kChunkBytes, &tmX, &mybar[b], c0, r0);
      }
    };
    if (MODE == MODE_AUX) issue_aux(0);

    uint32_t item = 0;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++tc) {
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
          if (lane == 0) mbar_arrive(&tempty[acc]);
        }
        const bool store_ok = (r0 < g.M) && (c0 < g.N);
        const bool full_cols = (c0 + 64 <= g.N);
        const int vo = g.batch_m_tiles ? (r0 / (kBM * g.batch_m_tiles)) * g.N : 0;   // offset of the problem's bias / scale
        // ---- x = (acc + bias) * scale
        if (g.bias) {
          if (full_cols && !(vo & 3)) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float4 b = __ldg(reinterpret_cast<const float4*>(g.bias + vo + c0) + j);
              v[4 * j] += b.x; v[4 * j + 1] += b.y; v[4 * j + 2] += b.z; v[4 * j + 3] += b.w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 64; ++j) if (c0 + j < g.N) v[j] += __ldg(g.bias + vo + c0 + j);
          }
        }
        if (g.scale && !g.scale_post) {
#pragma unroll
          for (int j = 0; j < 64; ++j) if (c0 + j < g.N) v[j] *= __ldg(g.scale + vo + c0 + j);
        }
        // ---- second output: pre-activation
        if (MODE == MODE_Z) {
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
        // ---- activation
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
          case ACT_SOFTMAX64: {
            float m = v[0];
#pragma unroll
            for (int j = 1; j < 64; ++j) m = fmaxf(m, v[j]);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 64; ++j) { v[j] = ex2_fast((v[j] - m) * 1.4426950409f); s += v[j]; }
            const float inv = __frcp_rn(s);
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] *= inv;
          } break;
          default: break;
        }
        // ---- auxiliary operand
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
            case AUX_DSOFTMAX: {
              float dot = 0.f;
#pragma unroll
              for (int j = 0; j < 64; ++j) dot += v[j] * a[j];
              float gs = 0.f;
#pragma unroll
              for (int j = 0; j < 64; ++j) {
                v[j] = a[j] * (v[j] - dot);
                gs += (a[j] > 0.f) ? v[j] * __logf(a[j]) : 0.f;
              }
              if (g.group_out) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) gs += __shfl_xor_sync(0xffffffffu, gs, o);
                if (lane == 0 && c0 < g.N) atomicAdd(g.group_out + (c0 >> 6), gs);
              }
            } break;
            default: break;
          }
        } else {
          if (lane == 0) tma_store_wait_read<NBUF - 1>();
          __syncwarp();
        }
        if (g.scale && g.scale_post) {
#pragma unroll
          for (int j = 0; j < 64; ++j) if (c0 + j < g.N) v[j] *= __ldg(g.scale + vo + c0 + j);
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
            if (r0 < g.M && c0 < g.N && yy < g.img_h) tma_store_4d(stg + b * kChunkBytes, &tmC, c0, x0, yy, n);
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
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------- host
struct GemmCall {
  const void* A; int lda;
  const void* A2; int lda2;
  const void* A3; int lda3;
  const void* B; int ldb;
  void* C; int ldc;
  void* Z; int ldz;          // optional second output (pre-activation)
  const void* AUX; int ldaux; // optional auxiliary input [M,N]
  int M, N, K, K1, K2;
  const float* bias; const float* scale; float* group_out;
  int act, aux_mode, scale_post;
  int max_ctas;  // 0 = number of SMs
  int split_m = 0;  // BN = 256 instantiation as 256-row x 128-column tiles (see GemmArgs::split_m)
  int batch = 1; // > 1: `batch` stacked problems (see GemmArgs::batch_m_tiles); M is the total row count, M / batch % 128 == 0
  // convolution: A is an NHWC image [img_n, img_h, img_w, cin], B holds [N, ksize*ksize*cin] (tap-major), C is NHWC
  int conv = 0, img_n = 0, img_h = 0, img_w = 0, cin = 0, ksize = 0;
  // halo exchange fused into the convolution (see GemmArgs): boundary rows published by the neighbours [img_n, 1, img_w, cin]
  int halo = 0;
  const void* up_rows = nullptr; const void* down_rows = nullptr;
  const uint32_t* flag_up = nullptr; const uint32_t* flag_down = nullptr;
  uint32_t halo_epoch = 0;
  double halo_budget_s = 0.0;   // 0 = the library default
};

template <int BN, int MODE>
inline int launch_gemm_tn(const GemmCall& c, int num_sms, int* err_word, cudaStream_t stream) {
  using Cfg = GemmCfg<BN, MODE>;
  CUtensorMap tA, tA2, tA3, tB, tC, tX;
  if (c.conv) {
    if (MODE != MODE_PLAIN) return -19;
    if (make_tmap_nhwc_b16(&tA, c.A, c.img_n, c.img_h, c.img_w, c.cin, kConvTileH, kConvTileW)) return -10;
    if (c.halo) {
      if (c.ksize != 3 || (c.img_h % kConvTileH)) return -20;
      if (make_tmap_nhwc_b16(&tA2, c.A, c.img_n, c.img_h, c.img_w, c.cin, kConvTileH - 1, kConvTileW)) return -11;
      if (c.up_rows && make_tmap_nhwc_b16(&tA3, c.up_rows, c.img_n, 1, c.img_w, c.cin, 1, kConvTileW)) return -18;
      if (c.down_rows && make_tmap_nhwc_b16(&tX, c.down_rows, c.img_n, 1, c.img_w, c.cin, 1, kConvTileW)) return -15;
    }
  } else if (make_tmap_2d_b16(&tA, c.A, c.M, c.K1, c.lda, kBM, kBK)) return -10;
  const bool halo = c.conv && c.halo;
  if (c.K2 > c.K1) { if (make_tmap_2d_b16(&tA2, c.A2, c.M, c.K2 - c.K1, c.lda2, kBM, kBK)) return -11; }
  else if (!halo) tA2 = tA;
  if (c.K > c.K2) { if (make_tmap_2d_b16(&tA3, c.A3, c.M, c.K - c.K2, c.lda3, kBM, kBK)) return -18; }
  else if (!(halo && c.up_rows)) tA3 = tA;
  if (c.batch > 1 && (c.conv || c.M % (c.batch * kBM) || c.group_out)) return -21;
  const bool split = BN == 256 && MODE == MODE_PLAIN && c.split_m && c.batch <= 1;
  if (make_tmap_2d_b16(&tB, c.B, c.N * (c.batch > 1 ? c.batch : 1), c.K, c.ldb, split ? 128 : BN, kBK)) return -12;
  if (c.conv) { if (make_tmap_nhwc_b16(&tC, c.C, c.img_n, c.img_h, c.img_w, c.N, 2, kConvTileW)) return -13; }
  else if (make_tmap_2d_b16(&tC, c.C, c.M, c.N, c.ldc, 32, 64)) return -13;
  if (MODE == MODE_Z) { if (make_tmap_2d_b16(&tX, c.Z, c.M, c.N, c.ldz, 32, 64)) return -14; }
  else if (MODE == MODE_AUX) { if (make_tmap_2d_b16(&tX, c.AUX, c.M, c.N, c.ldaux, 32, 64)) return -15; }
  else if (!(halo && c.down_rows)) tX = tC;
  GemmArgs g;
  g.M = c.M; g.N = c.N; g.K = c.K; g.K1 = c.K1; g.K2 = c.K2;
  g.bias = c.bias; g.scale = c.scale; g.group_out = c.group_out;
  g.act = c.act; g.aux_mode = c.aux_mode; g.scale_post = c.scale_post;
  g.num_m_tiles = (c.M + kBM - 1) / kBM;
  g.num_n_tiles = (c.N + BN - 1) / BN;
  g.err = err_word;
  g.batch_m_tiles = c.batch > 1 ? c.M / c.batch / kBM : 0;
  g.split_m = split ? 1 : 0;
  g.conv = c.conv; g.cin = c.cin; g.ksize = c.ksize; g.pad = c.ksize / 2; g.img_h = c.img_h;
  g.tiles_x = g.tiles_y = 0;
  g.halo = c.conv ? c.halo : 0; g.has_up = c.up_rows != nullptr; g.has_down = c.down_rows != nullptr; g.img_n = c.img_n;
  g.flag_up = c.flag_up; g.flag_down = c.flag_down; g.halo_epoch = c.halo_epoch;
  g.halo_budget_ns = c.halo_budget_s > 0.0 ? (unsigned long long)(c.halo_budget_s * 1e9) : kWaitBudgetNs;
  if (c.conv) {
    g.tiles_x = (c.img_w + kConvTileW - 1) / kConvTileW;
    g.tiles_y = (c.img_h + kConvTileH - 1) / kConvTileH;
    g.num_m_tiles = c.img_n * g.tiles_x * g.tiles_y;
    g.M = g.num_m_tiles * kBM;            // every row of a tile is "in range"; the copy engine clips at image edges
  }
  static unsigned long long attr_mask = 0;   // one bit per device: the attribute belongs to the device's context
  if (first_use_on_device(attr_mask)) {
    if (cudaFuncSetAttribute(gemm_tn_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) !=
        cudaSuccess)
      return -16;
  }
  if (split) {                                // 256-row tiles of 128 columns
    g.num_m_tiles = (g.num_m_tiles + 1) / 2;
    g.num_n_tiles = (c.N + 127) / 128;
  }
  int tiles = g.num_m_tiles * g.num_n_tiles;
  int cap = c.max_ctas > 0 ? c.max_ctas : num_sms;
  int grid = tiles < cap ? tiles : cap;
  gemm_tn_kernel<BN, MODE><<<grid, kGemmThreads, Cfg::SMEM, stream>>>(tA, tA2, tA3, tB, tC, tX, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -17;
}

}  // namespace pnm
