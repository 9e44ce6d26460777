// AFNO spectral filter with the token <-> channel resharding fused into its Fourier stages.
//
// The filter of one AFNO block is  irfft2( softshrink( blockMLP( rfft2(x)[kept modes] ) ) )  over the (H, W) grid of
// tokens, with a block-diagonal complex MLP that mixes the Cb channels of each of the model's blocks.  The token
// tensor x[t, C] (t = (b H + h) W + w) is sharded over the ranks by tokens for the LayerNorm / MLP part of the model;
// the filter needs whole (H, W) planes but only Cb channels at a time.  Each rank therefore OWNS some channel blocks,
// and the two reshardings are done by the Fourier kernels themselves:
//
//   rows   (grid: rows (b, h) x owned blocks)  pulls the 2 Cb-byte channel slice of every token of its row straight
//          from the token owners' memory (peer loads after a bounded wait on their flags) and computes the pruned
//          real-to-complex DFT along W (only the kept kx) -> Y[b, h, kx, c]
//   cols   (grid: (b, kx) x owned blocks)  DFT along H (two-level Cooley-Tukey in shared memory), the complex
//          two-layer MLP with ReLU, soft-shrink, inverse DFT along H -> Y'[b, h, kx, c]
//   rows^T (grid: rows x owned blocks)  complex-to-real inverse DFT along W and bf16 stores of the Cb-channel slice
//          of every token of the row INTO the token owner's memory (peer stores); the last block raises the flags
//
// so that no all-to-all, no transposed copy and no library FFT appear.  The backward runs the same three kernels
// with the adjoint weights (see the `kweight` arguments) and a column kernel that differentiates the MLP.
// All transforms are "ortho"-normalised, fp32 in shared memory; tokens are bf16.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "pnm_api.h"
#include "pnm_internal.h"

namespace pnm {

constexpr int kAfThreadsPerCh = 2;

struct TokenPtrs { __nv_bfloat16* p[kPeerMaxRanks]; };

struct AfGeom {
  int B, H, W, C;        // grid of tokens and total channels of a token row
  int Cb;                // channels per block (threads = 2 Cb)
  int KX;                // kept modes along W (kx = 0 .. KX-1, KX <= W/2)
  int blk0, nblk;        // first owned block and number of owned blocks
  long long Tp;          // tokens per rank (B H W = world * Tp)
  int H1, H2;            // factorisation H = H1 * H2 of the column transform
};

__device__ __forceinline__ const __nv_bfloat16* token_addr(const TokenPtrs& tp, const AfGeom& g, long long t, int c) {
  const int owner = int(t / g.Tp);
  return tp.p[owner] + (t - owner * g.Tp) * g.C + c;
}

// ---------------------------------------------------------------------------------------------------- rows: r2c
// Y[(row * KX + kx) * (nblk * Cb) + j * Cb + c] = kweight(kx) / sqrt(W) * sum_w x[row, w, blk c] e^{-2 pi i kx w / W}
// kweight: 0 -> 1 for every kx (forward);  1 -> 1 for kx = 0 and 2 otherwise (adjoint of the weighted c2r)
__global__ void __launch_bounds__(256)
afno_rows_r2c_kernel(TokenPtrs tok, float2* __restrict__ Y, AfGeom g, int kweight, PeerArgs peer, int wait, int* err) {
  extern __shared__ float sm[];
  __shared__ int sh_ok;
  float* x = sm;                                   // [W][Cb]
  float2* tw = reinterpret_cast<float2*>(x + (size_t)g.W * g.Cb);   // [W]
  const int row = blockIdx.x, j = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
  bool ok = true;
  if (wait) ok = peer_small_wait(peer, peer_epoch(peer), err, &sh_ok);
  for (int i = tid; i < g.W; i += nt) {
    float s, c;
    sincospif(2.f * i / g.W, &s, &c);
    tw[i] = make_float2(c, s);
  }
  const int c0 = (g.blk0 + j) * g.Cb;
  const int vec = g.Cb >> 3;                       // 16-byte vectors per token slice
  const float nanv = __int_as_float(0x7fc00000);
  for (int i = tid; i < g.W * vec; i += nt) {
    const int w = i / vec, v = i % vec;
    float f[8];
    if (ok) {
      const uint4 u = __ldcg(reinterpret_cast<const uint4*>(token_addr(tok, g, (long long)row * g.W + w, c0 + v * 8)));
      float2 a;
      a = unpack_bf16x2(u.x); f[0] = a.x; f[1] = a.y;
      a = unpack_bf16x2(u.y); f[2] = a.x; f[3] = a.y;
      a = unpack_bf16x2(u.z); f[4] = a.x; f[5] = a.y;
      a = unpack_bf16x2(u.w); f[6] = a.x; f[7] = a.y;
    } else {
      for (int q = 0; q < 8; ++q) f[q] = nanv;
    }
    for (int q = 0; q < 8; ++q) x[w * g.Cb + v * 8 + q] = f[q];
  }
  __syncthreads();
  const int c = tid % g.Cb, part = tid / g.Cb;
  if (part >= kAfThreadsPerCh) return;
  const float inv = rsqrtf((float)g.W);
  const int ldy = g.nblk * g.Cb;
  for (int kx = part; kx < g.KX; kx += kAfThreadsPerCh) {
    float re = 0.f, im = 0.f;
    int idx = 0;
    for (int w = 0; w < g.W; ++w) {
      const float xv = x[w * g.Cb + c];
      const float2 t = tw[idx];
      re += xv * t.x;
      im -= xv * t.y;
      idx += kx;
      if (idx >= g.W) idx -= g.W;
    }
    const float s = inv * ((kweight && kx > 0) ? 2.f : 1.f);
    Y[((size_t)row * g.KX + kx) * ldy + j * g.Cb + c] = make_float2(re * s, im * s);
  }
}

// ---------------------------------------------------------------------------------------------------- rows: c2r
// y[row, w, blk c] = 1 / sqrt(W) * sum_kx kweight(kx) Re( X[row, kx, c] e^{+2 pi i kx w / W} ), stored as bf16 into the
// owner of token (row, w).  kweight: 1 -> 1 for kx = 0 and 2 otherwise (inverse real transform); 0 -> 1 (adjoint of r2c)
__global__ void __launch_bounds__(256)
afno_rows_c2r_kernel(const float2* __restrict__ X, TokenPtrs tok, AfGeom g, int kweight, PeerArgs peer, int signal,
                     unsigned int* counter) {
  extern __shared__ float sm[];
  float2* xs = reinterpret_cast<float2*>(sm);                    // [KX][Cb]
  float2* tw = xs + (size_t)g.KX * g.Cb;                         // [W]
  __nv_bfloat16* ys = reinterpret_cast<__nv_bfloat16*>(tw + g.W);  // [W][Cb]
  const int row = blockIdx.x, j = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
  const int ldx = g.nblk * g.Cb;
  for (int i = tid; i < g.W; i += nt) {
    float s, c;
    sincospif(2.f * i / g.W, &s, &c);
    tw[i] = make_float2(c, s);
  }
  for (int i = tid; i < g.KX * g.Cb; i += nt) {
    const int kx = i / g.Cb, c = i % g.Cb;
    float2 v = X[((size_t)row * g.KX + kx) * ldx + j * g.Cb + c];
    const float s = (kweight && kx > 0) ? 2.f : 1.f;
    xs[i] = make_float2(v.x * s, v.y * s);
  }
  __syncthreads();
  const int c = tid % g.Cb, part = tid / g.Cb;
  if (part < kAfThreadsPerCh) {
    const float inv = rsqrtf((float)g.W);
    for (int w = part; w < g.W; w += kAfThreadsPerCh) {
      float acc = 0.f;
      int idx = 0;
      for (int kx = 0; kx < g.KX; ++kx) {
        const float2 v = xs[kx * g.Cb + c];
        const float2 t = tw[idx];
        acc += v.x * t.x - v.y * t.y;
        idx += w;
        if (idx >= g.W) idx -= g.W;
      }
      ys[w * g.Cb + c] = __float2bfloat16(acc * inv);
    }
  }
  __syncthreads();
  const int c0 = (g.blk0 + j) * g.Cb;
  const int vec = g.Cb >> 3;
  for (int i = tid; i < g.W * vec; i += nt) {
    const int w = i / vec, v = i % vec;
    const uint4 u = *reinterpret_cast<const uint4*>(ys + w * g.Cb + v * 8);
    *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(token_addr(tok, g, (long long)row * g.W + w, c0 + v * 8))) = u;
  }
  if (signal) {
    __threadfence_system();
    __syncthreads();
    if (tid == 0 && atomicAdd(counter, 1u) == gridDim.x * gridDim.y - 1) {
      *counter = 0;
      peer_small_publish(peer, peer_epoch(peer));
    }
  }
}

// ------------------------------------------------------------------------------------------ columns: DFT along H
// Two-level Cooley-Tukey on [H][Cb] complex data in shared memory, H = H1 * H2, one channel per thread pair.
// sign = -1: forward (e^{-i}), +1: inverse.  in -> tmp -> out (out may alias in).
__device__ __forceinline__ float2 cmul(float2 a, float2 b) { return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x); }

__device__ void col_dft(const float2* in, float2* tmp, float2* out, const float2* tw, int H, int H1, int H2, int Cb, float sign,
                        int c, int part) {
  // step 1: for every n2, an H1-point DFT over n1 (stride H2), times the twiddle W_H^{n2 k1}; tmp[k1 * H2 + n2]
  for (int n2 = part; n2 < H2; n2 += kAfThreadsPerCh) {
    for (int k1 = 0; k1 < H1; ++k1) {
      float2 acc = make_float2(0.f, 0.f);
      int idx = 0;                                   // (n1 * k1 * H2) mod H
      const int step = (k1 * H2) % H;
      for (int n1 = 0; n1 < H1; ++n1) {
        const float2 t = tw[idx];
        acc = make_float2(acc.x + in[(H2 * n1 + n2) * Cb + c].x * t.x - in[(H2 * n1 + n2) * Cb + c].y * (sign * t.y),
                          acc.y + in[(H2 * n1 + n2) * Cb + c].x * (sign * t.y) + in[(H2 * n1 + n2) * Cb + c].y * t.x);
        idx += step;
        if (idx >= H) idx -= H;
      }
      const float2 t = tw[(n2 * k1) % H];
      tmp[(k1 * H2 + n2) * Cb + c] = cmul(acc, make_float2(t.x, sign * t.y));
    }
  }
  __syncthreads();
  // step 2: for every k1, an H2-point DFT over n2; out[k1 + H1 * k2]
  const float inv = rsqrtf((float)H);
  for (int k1 = part; k1 < H1; k1 += kAfThreadsPerCh) {
    for (int k2 = 0; k2 < H2; ++k2) {
      float2 acc = make_float2(0.f, 0.f);
      int idx = 0;                                   // (n2 * k2 * H1) mod H
      const int step = (k2 * H1) % H;
      for (int n2 = 0; n2 < H2; ++n2) {
        const float2 v = tmp[(k1 * H2 + n2) * Cb + c];
        const float2 t = tw[idx];
        acc.x += v.x * t.x - v.y * (sign * t.y);
        acc.y += v.x * (sign * t.y) + v.y * t.x;
        idx += step;
        if (idx >= H) idx -= H;
      }
      out[(k1 + H1 * k2) * Cb + c] = make_float2(acc.x * inv, acc.y * inv);
    }
  }
  __syncthreads();
}

struct AfWeights {        // this rank's view of the filter parameters, fp32: w [2][nb][Cb][Cb], b [2][nb][Cb] (nb = all blocks)
  const float* w1; const float* b1; const float* w2; const float* b2;
  int nb;                 // number of blocks of the model (stride between the real and imaginary halves)
};

constexpr int kAfModes = 5;   // modes per register block of the MLP loops

// out[m][o] = sum_i ( xr[m][i] wr[i][o] - xi[m][i] wi[i][o] ) + br[o],  ( xi wr + xr wi ) + bi[o]  for the modes of `part`
__device__ void cmlp_layer(const float2* x, float2* out, const float* wr, const float* wi, const float* br, const float* bi, int M,
                           int Cb, int o, int part, bool relu) {
  const int per = (M + kAfThreadsPerCh - 1) / kAfThreadsPerCh;
  const int m_lo = part * per, m_hi = min(M, m_lo + per);
  for (int m0 = m_lo; m0 < m_hi; m0 += kAfModes) {
    float ar[kAfModes], ai[kAfModes];
#pragma unroll
    for (int q = 0; q < kAfModes; ++q) { ar[q] = br[o]; ai[q] = bi[o]; }
    for (int i = 0; i < Cb; ++i) {
      const float r = __ldg(wr + i * Cb + o), s = __ldg(wi + i * Cb + o);
#pragma unroll
      for (int q = 0; q < kAfModes; ++q) {
        if (m0 + q < m_hi) {
          const float2 v = x[(m0 + q) * Cb + i];
          ar[q] += v.x * r - v.y * s;
          ai[q] += v.y * r + v.x * s;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < kAfModes; ++q)
      if (m0 + q < m_hi) out[(m0 + q) * Cb + o] = relu ? make_float2(fmaxf(ar[q], 0.f), fmaxf(ai[q], 0.f)) : make_float2(ar[q], ai[q]);
  }
}

__device__ __forceinline__ float softshrink_f(float v, float l) { return v > l ? v - l : (v < -l ? v + l : 0.f); }

// grid (B * KX, nblk), 2 Cb threads.  Y: [B*H][KX][nblk*Cb] complex.  Saves Z (MLP input), O1 (after ReLU), O2 (after shrink),
// each [B*KX][nblk][H][Cb] complex, for the backward.  Yout has the layout of Y.
__global__ void __launch_bounds__(256)
afno_cols_fwd_kernel(const float2* __restrict__ Y, float2* __restrict__ Yout, float2* __restrict__ Zs, float2* __restrict__ O1s,
                     float2* __restrict__ O2s, AfWeights wt, AfGeom g, float lambda) {
  extern __shared__ float sm[];
  float2* a = reinterpret_cast<float2*>(sm);            // [H][Cb]
  float2* b = a + (size_t)g.H * g.Cb;                   // [H][Cb]
  float2* tw = b + (size_t)g.H * g.Cb;                  // [H]
  const int bk = blockIdx.x, j = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
  const int bb = bk / g.KX, kx = bk % g.KX;
  const int ld = g.nblk * g.Cb;
  for (int i = tid; i < g.H; i += nt) {
    float s, c;
    sincospif(2.f * i / g.H, &s, &c);
    tw[i] = make_float2(c, s);
  }
  for (int i = tid; i < g.H * g.Cb; i += nt) {
    const int h = i / g.Cb, c = i % g.Cb;
    a[i] = Y[((size_t)(bb * g.H + h) * g.KX + kx) * ld + j * g.Cb + c];
  }
  __syncthreads();
  const int c = tid % g.Cb, part = tid / g.Cb;
  col_dft(a, b, a, tw, g.H, g.H1, g.H2, g.Cb, -1.f, c, part);          // a = Z[ky][c]
  const size_t sbase = ((size_t)bk * g.nblk + j) * g.H * g.Cb;
  for (int i = tid; i < g.H * g.Cb; i += nt) Zs[sbase + i] = a[i];
  const int blk = g.blk0 + j;
  const size_t wsz = (size_t)g.Cb * g.Cb;
  const float* w1r = wt.w1 + (size_t)blk * wsz;
  const float* w1i = wt.w1 + ((size_t)wt.nb + blk) * wsz;
  const float* w2r = wt.w2 + (size_t)blk * wsz;
  const float* w2i = wt.w2 + ((size_t)wt.nb + blk) * wsz;
  cmlp_layer(a, b, w1r, w1i, wt.b1 + blk * g.Cb, wt.b1 + (wt.nb + blk) * g.Cb, g.H, g.Cb, c, part, true);
  __syncthreads();
  for (int i = tid; i < g.H * g.Cb; i += nt) O1s[sbase + i] = b[i];
  cmlp_layer(b, a, w2r, w2i, wt.b2 + blk * g.Cb, wt.b2 + (wt.nb + blk) * g.Cb, g.H, g.Cb, c, part, false);
  __syncthreads();
  for (int i = tid; i < g.H * g.Cb; i += nt) {
    const float2 v = a[i];
    const float2 s = make_float2(softshrink_f(v.x, lambda), softshrink_f(v.y, lambda));
    a[i] = s;
    O2s[sbase + i] = s;
  }
  __syncthreads();
  col_dft(a, b, a, tw, g.H, g.H1, g.H2, g.Cb, +1.f, c, part);
  for (int i = tid; i < g.H * g.Cb; i += nt) {
    const int h = i / g.Cb, cc = i % g.Cb;
    Yout[((size_t)(bb * g.H + h) * g.KX + kx) * ld + j * g.Cb + cc] = a[i];
  }
}

// g[m][i] = sum_o ( dr[m][o] wr[i][o] + di[m][o] wi[i][o] ),  ( -dr[m][o] wi[i][o] + di[m][o] wr[i][o] ): the transposed
// complex product (adjoint of cmlp_layer without bias) for input channel i of this thread
__device__ void cmlp_layer_t(const float2* d, float2* out, const float* wr, const float* wi, int M, int Cb, int i, int part) {
  const int per = (M + kAfThreadsPerCh - 1) / kAfThreadsPerCh;
  const int m_lo = part * per, m_hi = min(M, m_lo + per);
  for (int m0 = m_lo; m0 < m_hi; m0 += kAfModes) {
    float ar[kAfModes], ai[kAfModes];
#pragma unroll
    for (int q = 0; q < kAfModes; ++q) ar[q] = ai[q] = 0.f;
    for (int o = 0; o < Cb; ++o) {
      const float r = __ldg(wr + i * Cb + o), s = __ldg(wi + i * Cb + o);
#pragma unroll
      for (int q = 0; q < kAfModes; ++q) {
        if (m0 + q < m_hi) {
          const float2 v = d[(m0 + q) * Cb + o];
          ar[q] += v.x * r + v.y * s;
          ai[q] += -v.x * s + v.y * r;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < kAfModes; ++q)
      if (m0 + q < m_hi) out[(m0 + q) * Cb + i] = make_float2(ar[q], ai[q]);
  }
}

// dW[i][o] (real, imag) += sum_m x[m][i] (*) g[m][o] with the pairing of cmlp_layer:  dWr += xr gr + xi gi ; dWi += -xi gr + xr gi
// thread = output channel o (part 0) ; loops over i; atomics into the global gradient (shared by all (b, kx) CTAs)
__device__ void cmlp_wgrad(const float2* x, const float2* gr, float* dwr, float* dwi, float* dbr, float* dbi, int M, int Cb, int o,
                           int part) {
  for (int i = part; i < Cb; i += kAfThreadsPerCh) {
    float a = 0.f, b = 0.f;
    for (int m = 0; m < M; ++m) {
      const float2 xv = x[m * Cb + i], gv = gr[m * Cb + o];
      a += xv.x * gv.x + xv.y * gv.y;
      b += -xv.y * gv.x + xv.x * gv.y;
    }
    atomicAdd(dwr + i * Cb + o, a);
    atomicAdd(dwi + i * Cb + o, b);
  }
  if (part == 0) {
    float a = 0.f, b = 0.f;
    for (int m = 0; m < M; ++m) { a += gr[m * Cb + o].x; b += gr[m * Cb + o].y; }
    atomicAdd(dbr + o, a);
    atomicAdd(dbi + o, b);
  }
}

struct AfGrads { float* dw1; float* db1; float* dw2; float* db2; };

// Backward of afno_cols_fwd_kernel.  dYout: gradient w.r.t. Yout (layout of Y); dY: gradient w.r.t. Y.
__global__ void __launch_bounds__(256)
afno_cols_bwd_kernel(const float2* __restrict__ dYout, float2* __restrict__ dY, const float2* __restrict__ Zs,
                     const float2* __restrict__ O1s, const float2* __restrict__ O2s, AfWeights wt, AfGrads gd, AfGeom g) {
  extern __shared__ float sm[];
  float2* a = reinterpret_cast<float2*>(sm);            // [H][Cb]
  float2* b = a + (size_t)g.H * g.Cb;
  float2* x = b + (size_t)g.H * g.Cb;                   // saved activation of the layer being differentiated
  float2* tw = x + (size_t)g.H * g.Cb;
  const int bk = blockIdx.x, j = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
  const int bb = bk / g.KX, kx = bk % g.KX;
  const int ld = g.nblk * g.Cb;
  for (int i = tid; i < g.H; i += nt) {
    float s, c;
    sincospif(2.f * i / g.H, &s, &c);
    tw[i] = make_float2(c, s);
  }
  for (int i = tid; i < g.H * g.Cb; i += nt) {
    const int h = i / g.Cb, c = i % g.Cb;
    a[i] = dYout[((size_t)(bb * g.H + h) * g.KX + kx) * ld + j * g.Cb + c];
  }
  __syncthreads();
  const int c = tid % g.Cb, part = tid / g.Cb;
  col_dft(a, b, a, tw, g.H, g.H1, g.H2, g.Cb, -1.f, c, part);          // adjoint of the inverse DFT: a = d O2(shrunk)
  const size_t sbase = ((size_t)bk * g.nblk + j) * g.H * g.Cb;
  for (int i = tid; i < g.H * g.Cb; i += nt) {                          // soft-shrink mask; load O1 (input of layer 2)
    const float2 s = O2s[sbase + i];
    a[i] = make_float2(s.x != 0.f ? a[i].x : 0.f, s.y != 0.f ? a[i].y : 0.f);
    x[i] = O1s[sbase + i];
  }
  __syncthreads();
  const int blk = g.blk0 + j;
  const size_t wsz = (size_t)g.Cb * g.Cb;
  cmlp_wgrad(x, a, gd.dw2 + (size_t)blk * wsz, gd.dw2 + ((size_t)wt.nb + blk) * wsz, gd.db2 + blk * g.Cb,
             gd.db2 + (wt.nb + blk) * g.Cb, g.H, g.Cb, c, part);
  cmlp_layer_t(a, b, wt.w2 + (size_t)blk * wsz, wt.w2 + ((size_t)wt.nb + blk) * wsz, g.H, g.Cb, c, part);   // b = d O1
  __syncthreads();
  for (int i = tid; i < g.H * g.Cb; i += nt) {                          // ReLU mask (x still holds O1); then load Z
    const float2 o1 = x[i];
    b[i] = make_float2(o1.x > 0.f ? b[i].x : 0.f, o1.y > 0.f ? b[i].y : 0.f);
  }
  __syncthreads();
  for (int i = tid; i < g.H * g.Cb; i += nt) x[i] = Zs[sbase + i];
  __syncthreads();
  cmlp_wgrad(x, b, gd.dw1 + (size_t)blk * wsz, gd.dw1 + ((size_t)wt.nb + blk) * wsz, gd.db1 + blk * g.Cb,
             gd.db1 + (wt.nb + blk) * g.Cb, g.H, g.Cb, c, part);
  cmlp_layer_t(b, a, wt.w1 + (size_t)blk * wsz, wt.w1 + ((size_t)wt.nb + blk) * wsz, g.H, g.Cb, c, part);   // a = d Z
  __syncthreads();
  col_dft(a, b, a, tw, g.H, g.H1, g.H2, g.Cb, +1.f, c, part);          // adjoint of the forward DFT
  for (int i = tid; i < g.H * g.Cb; i += nt) {
    const int h = i / g.Cb, cc = i % g.Cb;
    dY[((size_t)(bb * g.H + h) * g.KX + kx) * ld + j * g.Cb + cc] = a[i];
  }
}

static TokenPtrs make_tok(const void* const* ptrs) {
  TokenPtrs t;
  for (int r = 0; r < kPeerMaxRanks; ++r) t.p[r] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(ptrs[r]));
  return t;
}

static int af_check(const AfGeom& g) {
  if (g.B <= 0 || g.H <= 0 || g.W <= 0 || g.Cb <= 0 || g.Cb % 8 || 2 * g.Cb > 256 || g.KX <= 0 || 2 * g.KX > g.W + 1 || g.nblk <= 0 ||
      g.H1 * g.H2 != g.H || g.Tp <= 0 || g.C % 8)
    return -2;
  return 0;
}

template <typename K>
static int af_smem_attr(K kernel, size_t bytes, unsigned long long& mask) {
  if (bytes > 220 * 1024) return -2;
  if (first_use_on_device(mask) && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
    return -4;
  return 0;
}

}  // namespace pnm

extern "C" {

// geom: {B, H, W, C, Cb, KX, blk0, nblk, H1, H2} ints; Tp tokens per rank.  tokens: host array of 8 (peer-mapped) addresses of
// the ranks' token buffers [Tp, C] bf16 (unused entries repeat a valid one).
int pnm_afno_rows_r2c(const void* const* tokens, void* Y, const int* geom, long long Tp, int kweight, int wait,
                      const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s,
                      const void* epoch_base, void* stream) {
  pnm::AfGeom g{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], Tp, geom[8], geom[9]};
  if (pnm::af_check(g)) return -2;
  int* err = pnm::error_word_ptr();
  if (!err) return -1;
  const size_t smem = sizeof(float) * ((size_t)g.W * g.Cb + 2 * g.W);
  static unsigned long long mask = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_rows_r2c_kernel, smem, mask)) return rc;
  pnm::PeerArgs p{};
  if (wait) p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  pnm::afno_rows_r2c_kernel<<<dim3(g.B * g.H, g.nblk), 2 * g.Cb, smem, (cudaStream_t)stream>>>(pnm::make_tok(tokens), (float2*)Y, g,
                                                                                              kweight, p, wait, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// signal != 0: after all stores the last block raises this rank's flags of call `epoch` (counter: zeroed device uint32).
int pnm_afno_rows_c2r(const void* X, const void* const* tokens, const int* geom, long long Tp, int kweight, int signal,
                      const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats,
                      const void* epoch_base, void* counter, void* stream) {
  pnm::AfGeom g{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], Tp, geom[8], geom[9]};
  if (pnm::af_check(g) || (signal && !counter)) return -2;
  const size_t smem = sizeof(float2) * ((size_t)g.KX * g.Cb + g.W) + sizeof(__nv_bfloat16) * (size_t)g.W * g.Cb;
  static unsigned long long mask = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_rows_c2r_kernel, smem, mask)) return rc;
  pnm::PeerArgs p{};
  if (signal) p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, 1.0, epoch_base);
  pnm::afno_rows_c2r_kernel<<<dim3(g.B * g.H, g.nblk), 2 * g.Cb, smem, (cudaStream_t)stream>>>((const float2*)X, pnm::make_tok(tokens),
                                                                                              g, kweight, p, signal,
                                                                                              (unsigned int*)counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// w1 / b1 / w2 / b2: the filter parameters of the whole model ([2, nb, Cb, Cb] / [2, nb, Cb], fp32); saved: Z, O1, O2
// each [B*KX, nblk, H, Cb] complex64.
int pnm_afno_cols_fwd(const void* Y, void* Yout, void* Zs, void* O1s, void* O2s, const float* w1, const float* b1, const float* w2,
                      const float* b2, int nb, const int* geom, float lambda, void* stream) {
  pnm::AfGeom g{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], 1, geom[8], geom[9]};
  if (pnm::af_check(g) || nb < g.blk0 + g.nblk) return -2;
  const size_t smem = sizeof(float2) * (2 * (size_t)g.H * g.Cb + g.H);
  static unsigned long long mask = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_cols_fwd_kernel, smem, mask)) return rc;
  pnm::AfWeights wt{w1, b1, w2, b2, nb};
  pnm::afno_cols_fwd_kernel<<<dim3(g.B * g.KX, g.nblk), 2 * g.Cb, smem, (cudaStream_t)stream>>>(
      (const float2*)Y, (float2*)Yout, (float2*)Zs, (float2*)O1s, (float2*)O2s, wt, g, lambda);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dw1 / db1 / dw2 / db2 (layouts of the parameters) are ACCUMULATED into with atomics.
int pnm_afno_cols_bwd(const void* dYout, void* dY, const void* Zs, const void* O1s, const void* O2s, const float* w1, const float* w2,
                      float* dw1, float* db1, float* dw2, float* db2, int nb, const int* geom, void* stream) {
  pnm::AfGeom g{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], 1, geom[8], geom[9]};
  if (pnm::af_check(g) || nb < g.blk0 + g.nblk) return -2;
  const size_t smem = sizeof(float2) * (3 * (size_t)g.H * g.Cb + g.H);
  static unsigned long long mask = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_cols_bwd_kernel, smem, mask)) return rc;
  pnm::AfWeights wt{w1, nullptr, w2, nullptr, nb};
  pnm::AfGrads gd{dw1, db1, dw2, db2};
  pnm::afno_cols_bwd_kernel<<<dim3(g.B * g.KX, g.nblk), 2 * g.Cb, smem, (cudaStream_t)stream>>>(
      (const float2*)dYout, (float2*)dY, (const float2*)Zs, (const float2*)O1s, (const float2*)O2s, wt, gd, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
