// LayerNorm forward / backward over the last dimension, bf16 activations, fp32 statistics
// and parameters.  One warp per row, 16-byte vector loads, persistent grid-stride loop so
// that the per-column reductions of the backward (dgamma, dbeta) stay in registers until
// the CTA writes one partial row to scratch; a second tiny kernel folds the partials.
#pragma once
#include "common.cuh"

namespace pnm {

constexpr int kLnWarps = 8;
constexpr int kLnMaxVec = 4;  // supports C up to 32 lanes * 8 elems * 4 = 1024

// y = (x - mean) * rstd * gamma + beta (+ post); optional second input r: normalises (x + r)
// and writes the sum to `sum_out` (fused residual add before the normalisation).
// LPR lanes share a row: 32 (one row per warp) or 16 (two rows per warp, C <= 256).  With a whole warp on a 256-wide row
// the kernel is bound by instruction issue, not by memory (ncu: warps stall "not selected" / on the shuffle chains while
// DRAM is ~50 % busy); two rows per warp halve the instructions per row.
template <int VEC, bool HAS_R, int LPR = 32>
__global__ void __launch_bounds__(kLnWarps * 32, VEC == 1 ? 3 : 2)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ r_in,
                     const float* __restrict__ gamma, const float* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                     __nv_bfloat16* __restrict__ sum_out, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                     const __nv_bfloat16* __restrict__ post, long long M, int C, float eps) {
  constexpr int RW = 32 / LPR;                            // rows per warp and step
  const __nv_bfloat16* r = HAS_R ? r_in : nullptr;      // without the second input its ring of registers disappears
  const int lane = threadIdx.x & 31, l = lane % LPR, sub = lane / LPR;
  const long long first = ((long long)blockIdx.x * kLnWarps + (threadIdx.x >> 5)) * RW + sub;
  const long long stride = (long long)gridDim.x * kLnWarps * RW;
  float gam[VEC][8], bet[VEC][8];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    const int c = (v * LPR + l) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gam[v][j] = (c + j < C) ? gamma[c + j] : 0.f;
      bet[v][j] = (c + j < C && beta) ? beta[c + j] : 0.f;
    }
  }
  // A ring of D steps per warp is kept in flight: the loads of step i + D are issued before step i is processed.
  constexpr int D = (VEC <= 2) ? 2 : 1;                  // wider rows: the ring would spill
  uint4 nx[D][VEC], nr[D][VEC];
  auto fetch = [&](int slot, long long row) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int c = (v * LPR + l) * 8;
      const bool live = row < M && c < C;
      nx[slot][v] = live ? *reinterpret_cast<const uint4*>(x + row * C + c) : make_uint4(0u, 0u, 0u, 0u);
      if (HAS_R) nr[slot][v] = live ? *reinterpret_cast<const uint4*>(r + row * C + c) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
#pragma unroll
  for (int d = 0; d < D; ++d) fetch(d, first + d * stride);
  // the loop bound is the same for all lanes of a warp (the shuffles below need every lane): rows past M are masked
  for (long long row0 = first - sub; row0 < M; row0 += D * stride) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
      const long long row = row0 + sub + d * stride;
      const bool in = row < M;
      if (row0 + d * stride >= M) break;
      float val[VEC][8];
      float s = 0.f;
      uint4 cx[VEC], cr[VEC];
#pragma unroll
      for (int v = 0; v < VEC; ++v) { cx[v] = nx[d][v]; if (HAS_R) cr[v] = nr[d][v]; }
      fetch(d, row + D * stride);
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        const int c = (v * LPR + l) * 8;
        if (c < C) {
          const uint4 u = cx[v];
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
          uint32_t rw[4] = {0, 0, 0, 0};
          if (HAS_R) {
            const uint4 ur = cr[v];
            rw[0] = ur.x; rw[1] = ur.y; rw[2] = ur.z; rw[3] = ur.w;
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = unpack_bf16x2(w[j]);
            if (HAS_R) { float2 fr = unpack_bf16x2(rw[j]); f.x += fr.x; f.y += fr.y; }
            val[v][2 * j] = f.x; val[v][2 * j + 1] = f.y;
            s += f.x + f.y;
          }
          if (HAS_R && sum_out && in) {
            uint4 o;
            o.x = pack_bf16x2(val[v][0], val[v][1]); o.y = pack_bf16x2(val[v][2], val[v][3]);
            o.z = pack_bf16x2(val[v][4], val[v][5]); o.w = pack_bf16x2(val[v][6], val[v][7]);
            *reinterpret_cast<uint4*>(sum_out + row * C + c) = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) val[v][j] = 0.f;
        }
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s / C;
      float sq = 0.f;
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        const int c = (v * LPR + l) * 8;
        if (c < C) {
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float dd = val[v][j] - mean; sq += dd * dd; }
        }
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      const float rstd = rsqrtf(sq / C + eps);
      if (l == 0 && in) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
      }
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        const int c = (v * LPR + l) * 8;
        if (c < C && in) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = (val[v][j] - mean) * rstd * gam[v][j] + bet[v][j];
          if (post) {  // y = LN(x) + post  (residual added after the normalisation)
            const uint4 up = *reinterpret_cast<const uint4*>(post + row * C + c);
            float2 f;
            f = unpack_bf16x2(up.x); o[0] += f.x; o[1] += f.y;
            f = unpack_bf16x2(up.y); o[2] += f.x; o[3] += f.y;
            f = unpack_bf16x2(up.z); o[4] += f.x; o[5] += f.y;
            f = unpack_bf16x2(up.w); o[6] += f.x; o[7] += f.y;
          }
          uint4 u;
          u.x = pack_bf16x2(o[0], o[1]); u.y = pack_bf16x2(o[2], o[3]);
          u.z = pack_bf16x2(o[4], o[5]); u.w = pack_bf16x2(o[6], o[7]);
          *reinterpret_cast<uint4*>(y + row * C + c) = u;
        }
      }
    }
  }
}

// dx = rstd * (g*dy - mean_c(g*dy) - xhat * mean_c(g*dy*xhat)) (+ dres) ; partial dgamma/dbeta
// rows go to scratch[blockIdx.x][2][C].  LPR as in the forward kernel.
template <int VEC, int LPR = 32>
__global__ void __launch_bounds__(kLnWarps * 32, (VEC == 1 && LPR == 32) ? 3 : (LPR == 16 ? 2 : 1))
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const float* __restrict__ gamma, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ scratch, long long M, int C) {
  constexpr int RW = 32 / LPR;
  constexpr int COLS = LPR * 8;                           // columns one vector slot covers
  __shared__ float red[kLnWarps][2][32 * 8 + 8];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, l = lane % LPR, sub = lane / LPR;
  const long long first = ((long long)blockIdx.x * kLnWarps + wib) * RW + sub;
  const long long stride = (long long)gridDim.x * kLnWarps * RW;
  float gam[VEC][8], dg[VEC][8], db[VEC][8];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    const int c = (v * LPR + l) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gam[v][j] = (c + j < C) ? gamma[c + j] : 0.f;
      dg[v][j] = 0.f; db[v][j] = 0.f;
    }
  }
  // x, dy and the residual gradient of the next D steps are requested before a step is processed.  Measured at C = 256,
  // 1 M rows: D = 1 at three CTAs per SM 0.45 ms; D = 2 at three CTAs (80 registers, spills) 0.79 ms; two rows per warp
  // (LPR = 16, two CTAs) 0.45 ms; D = 3 at two CTAs spills as well.  ncu: long-scoreboard stalls dominate (DRAM 51 % busy).
  constexpr int D = 1;
  uint4 nx[D][VEC], nd[D][VEC], nr[D][VEC];
  float nmean[D], nrstd[D];
  auto fetch = [&](int slot, long long row) {
    const bool in = row < M;
    nmean[slot] = in ? mean_in[row] : 0.f;
    nrstd[slot] = in ? rstd_in[row] : 0.f;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int c = (v * LPR + l) * 8;
      const bool live = in && c < C;
      nx[slot][v] = live ? *reinterpret_cast<const uint4*>(x + row * C + c) : make_uint4(0u, 0u, 0u, 0u);
      nd[slot][v] = live ? *reinterpret_cast<const uint4*>(dy + row * C + c) : make_uint4(0u, 0u, 0u, 0u);
      nr[slot][v] = (live && dres) ? *reinterpret_cast<const uint4*>(dres + row * C + c) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
#pragma unroll
  for (int d = 0; d < D; ++d) fetch(d, first + d * stride);
  // the loop bound is the same for all lanes of a warp; rows past M carry zeros and are not stored
  for (long long row00 = first - sub; row00 < M; row00 += D * stride) {
#pragma unroll
  for (int d = 0; d < D; ++d) {
    const long long row0 = row00 + d * stride;
    if (row0 >= M) break;
    const long long row = row0 + sub;
    const bool in = row < M;
    const float mean = nmean[d], rstd = nrstd[d];
    float xh[VEC][8], gy[VEC][8];
    uint4 ur[VEC], cx[VEC], cd[VEC];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < VEC; ++v) { ur[v] = nr[d][v]; cx[v] = nx[d][v]; cd[v] = nd[d][v]; }
    fetch(d, row + D * stride);
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int c = (v * LPR + l) * 8;
      if (c < C) {
        const uint4 ux = cx[v];
        const uint4 ud = cd[v];
        const uint32_t wx[4] = {ux.x, ux.y, ux.z, ux.w}, wd[4] = {ud.x, ud.y, ud.z, ud.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 fx = unpack_bf16x2(wx[j]), fd = unpack_bf16x2(wd[j]);
          const float h0 = (fx.x - mean) * rstd, h1 = (fx.y - mean) * rstd;   // rows past M: x = dy = 0, rstd = 0
          xh[v][2 * j] = h0; xh[v][2 * j + 1] = h1;
          dg[v][2 * j] += fd.x * h0; dg[v][2 * j + 1] += fd.y * h1;
          db[v][2 * j] += fd.x; db[v][2 * j + 1] += fd.y;
          const float g0 = fd.x * gam[v][2 * j], g1 = fd.y * gam[v][2 * j + 1];
          gy[v][2 * j] = g0; gy[v][2 * j + 1] = g1;
          s1 += g0 + g1; s2 += g0 * h0 + g1 * h1;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { xh[v][j] = 0.f; gy[v][j] = 0.f; }
      }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const float m1 = s1 / C, m2 = s2 / C;
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const int c = (v * LPR + l) * 8;
      if (c < C && in) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (gy[v][j] - m1 - xh[v][j] * m2);
        if (dres) {
          const uint32_t wr[4] = {ur[v].x, ur[v].y, ur[v].z, ur[v].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(wr[j]); o[2 * j] += f.x; o[2 * j + 1] += f.y; }
        }
        uint4 u;
        u.x = pack_bf16x2(o[0], o[1]); u.y = pack_bf16x2(o[2], o[3]);
        u.z = pack_bf16x2(o[4], o[5]); u.w = pack_bf16x2(o[6], o[7]);
        *reinterpret_cast<uint4*>(dx + row * C + c) = u;
      }
    }
  }
  }
  // fold the row halves of a warp, then the warps of this CTA, one vector slot at a time, and write the CTA partial
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = dg[v][j], b = db[v][j];
      if (LPR == 16) { a += __shfl_xor_sync(0xffffffffu, a, 16); b += __shfl_xor_sync(0xffffffffu, b, 16); }
      if (sub == 0) { red[wib][0][l * 8 + j] = a; red[wib][1][l * 8 + j] = b; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * COLS; i += kLnWarps * 32) {
      const int which = i / COLS, col = i % COLS;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kLnWarps; ++w) s += red[w][which][col];
      const int c = v * COLS + col;
      if (c < C) scratch[((size_t)blockIdx.x * 2 + which) * C + c] = s;
    }
    __syncthreads();
  }
}

// dgamma[c] = sum_b scratch[b][0][c], dbeta[c] = sum_b scratch[b][1][c].  A CTA owns 32 consecutive entries of the
// 2 C-wide scratch row; its 16 row groups walk the nblocks rows in parallel (coalesced 128-byte reads) and are folded
// through shared memory, so the dependent chain is nblocks / 16 loads instead of nblocks.
constexpr int kLnFoldRows = 16;
static __global__ void __launch_bounds__(32 * kLnFoldRows)
layernorm_bwd_finalize_kernel(const float* __restrict__ scratch, int nblocks, int C, float* __restrict__ dgamma,
                              float* __restrict__ dbeta) {
  __shared__ float part[kLnFoldRows][33];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;                       // entry of the [2][C] row
  float s = 0.f;
  if (i < 2 * C)
    for (int b = grp; b < nblocks; b += kLnFoldRows) s += scratch[(size_t)b * 2 * C + i];
  part[grp][lane] = s;
  __syncthreads();
  if (grp == 0 && i < 2 * C) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < kLnFoldRows; ++g) t += part[g][lane];
    const int which = i / C, c = i % C;
    if (which == 0) { if (dgamma) dgamma[c] = t; }
    else { if (dbeta) dbeta[c] = t; }
  }
}

inline int ln_vec_for(int C) { return (C + 255) / 256; }

inline int launch_layernorm_fwd(const void* x, const void* r, const float* gamma, const float* beta, void* y,
                                void* sum_out, float* mean, float* rstd, const void* post, long long M, int C,
                                float eps, int num_sms, cudaStream_t st) {
  if (C % 8 || C > 1024) return -30;
  long long want = (M + kLnWarps - 1) / kLnWarps;
  // whole waves of resident CTAs (3 per SM for C <= 128, 2 above): a partial last wave would idle part of the SMs
  const long long resident = (long long)num_sms * (C <= 128 ? 3 : 2);
  int grid = (int)(want < resident * 2 ? want : resident * 2);
  if (grid < 1) grid = 1;
  auto X = (const __nv_bfloat16*)x; auto R = (const __nv_bfloat16*)r; auto Y = (__nv_bfloat16*)y; auto S = (__nv_bfloat16*)sum_out; auto P = (const __nv_bfloat16*)post;
#define PNM_LN_FWD(V, L)                                                                                                   \
  if (R) layernorm_fwd_kernel<V, true, L><<<grid, kLnWarps * 32, 0, st>>>(X, R, gamma, beta, Y, S, mean, rstd, P, M, C, eps); \
  else layernorm_fwd_kernel<V, false, L><<<grid, kLnWarps * 32, 0, st>>>(X, R, gamma, beta, Y, S, mean, rstd, P, M, C, eps)
  if (C <= 128) { PNM_LN_FWD(1, 16); }
  else if (C <= 256) { PNM_LN_FWD(2, 16); }
  else if (C <= 512) { PNM_LN_FWD(2, 32); }
  else if (C <= 768) { PNM_LN_FWD(3, 32); }
  else { PNM_LN_FWD(4, 32); }
#undef PNM_LN_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -31;
}

// Number of CTAs the backward uses (= rows of scratch needed: grid * 2 * C floats).
// Grid of the backward kernel: whole waves of (at most) three resident CTAs per SM.
inline int layernorm_bwd_grid(long long M, int num_sms, int C = 0) {
  (void)C;
  long long want = (M + kLnWarps - 1) / kLnWarps;
  const int per_sm = 3;
  int grid = (int)(want < (long long)num_sms * per_sm ? want : (long long)num_sms * per_sm);
  return grid < 1 ? 1 : grid;
}

inline int launch_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean,
                                const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta,
                                float* scratch, long long M, int C, int num_sms, cudaStream_t st) {
  if (C % 8 || C > 1024) return -32;
  const int grid = layernorm_bwd_grid(M, num_sms, C);
  auto DY = (const __nv_bfloat16*)dy; auto X = (const __nv_bfloat16*)x; auto DR = (const __nv_bfloat16*)dres; auto DX = (__nv_bfloat16*)dx;
  if (C <= 256) layernorm_bwd_kernel<1><<<grid, kLnWarps * 32, 0, st>>>(DY, X, gamma, mean, rstd, DR, DX, scratch, M, C);
  else if (C <= 512) layernorm_bwd_kernel<2><<<grid, kLnWarps * 32, 0, st>>>(DY, X, gamma, mean, rstd, DR, DX, scratch, M, C);
  else if (C <= 768) layernorm_bwd_kernel<3><<<grid, kLnWarps * 32, 0, st>>>(DY, X, gamma, mean, rstd, DR, DX, scratch, M, C);
  else layernorm_bwd_kernel<4><<<grid, kLnWarps * 32, 0, st>>>(DY, X, gamma, mean, rstd, DR, DX, scratch, M, C);
  if (cudaGetLastError() != cudaSuccess) return -33;
  layernorm_bwd_finalize_kernel<<<(2 * C + 31) / 32, 32 * kLnFoldRows, 0, st>>>(scratch, grid, C, dgamma, dbeta);
  return cudaGetLastError() == cudaSuccess ? 0 : -34;
}

}  // namespace pnm
