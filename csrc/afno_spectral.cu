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

__device__ __forceinline__ void sm_unpack8(const uint4& u, float* f) {
  float2 a;
  a = unpack_bf16x2(u.x); f[0] = a.x; f[1] = a.y;
  a = unpack_bf16x2(u.y); f[2] = a.x; f[3] = a.y;
  a = unpack_bf16x2(u.z); f[4] = a.x; f[5] = a.y;
  a = unpack_bf16x2(u.w); f[6] = a.x; f[7] = a.y;
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


// ------------------------------------------------------------------------- rows, register-blocked form (W even)
// The same two transforms at several times the arithmetic rate of the kernels above, which issue two shared loads and
// an index update for every multiply-add pair.  Three changes:
//   * real-input symmetry: with e[w] = x[w] + x[W-w] and o[w] = x[w] - x[W-w] (w = 1 .. W/2-1),
//       Re X[k] = x[0] + (-1)^k x[W/2] + sum_w e[w] cos(2 pi k w / W),   Im X[k] = - sum_w o[w] sin(2 pi k w / W),
//     and in the other direction y[w] = A[w] - B[w], y[W-w] = A[w] + B[w] from the cosine / sine sums: half the work;
//   * a thread owns TWO adjacent channels and kRowNK modes (positions), so a twiddle fetched from shared memory
//     (a [w][k] table with the product index already reduced mod W, read as 16-byte vectors) feeds eight
//     multiply-adds and the x / X operands are reused kRowNK times from registers;
//   * 4 kRowNK independent accumulators per thread hide the multiply-add latency without more warps.
constexpr int kRowNK = 6;

struct RowPlan { int groups, passes, pad, threads; };

static RowPlan row_plan(int n_items, int cb) {
  const int cp = cb / 2;
  const int blocks = (n_items + kRowNK - 1) / kRowNK;
  const int max_groups = 512 / cp > 0 ? 512 / cp : 1;
  RowPlan p;
  p.passes = (blocks + max_groups - 1) / max_groups;
  p.groups = (blocks + p.passes - 1) / p.passes;
  p.pad = p.passes * p.groups * kRowNK;
  p.threads = ((cp * p.groups + 31) / 32) * 32;
  if (p.threads < 128) p.threads = 128;
  return p;
}

__global__ void __launch_bounds__(512)
afno_rows_r2c_v2_kernel(TokenPtrs tok, float2* __restrict__ Y, AfGeom g, int kweight, PeerArgs peer, int wait, int* err, int groups,
                        int passes) {
  extern __shared__ float sm[];
  __shared__ int sh_ok;
  const int Wh = g.W >> 1, nfold = Wh - 1, CP = g.Cb >> 1;
  const int pad = passes * groups * kRowNK;
  float* xe = sm;                                    // [nfold][Cb]
  float* xo = xe + (size_t)nfold * g.Cb;             // [nfold][Cb]
  float* x0 = xo + (size_t)nfold * g.Cb;             // [Cb]   sample w = 0
  float* xh = x0 + g.Cb;                             // [Cb]   sample w = W/2
  float2* tw2 = reinterpret_cast<float2*>(xh + g.Cb);   // [nfold][pad]: (cos, sin)(2 pi ((k w) mod W) / W), w = row + 1
  const int row = blockIdx.x, j = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
  bool ok = true;
  if (wait) ok = peer_small_wait(peer, peer_epoch(peer), err, &sh_ok);
  for (int i = tid; i < nfold * pad; i += nt) {
    const int w = i / pad + 1, k = i % pad;
    float sn, cs;
    sincospif(2.f * ((k * w) % g.W) / g.W, &sn, &cs);
    tw2[i] = make_float2(cs, sn);
  }
  const int c0 = (g.blk0 + j) * g.Cb;
  const int vec = g.Cb >> 3;
  const float nanv = __int_as_float(0x7fc00000);
  for (int i = tid; i < (Wh + 1) * vec; i += nt) {
    const int w = i / vec, v = i % vec;
    float f[8], h[8];
    const bool pair = w > 0 && w < Wh;
    if (ok) {
      sm_unpack8(__ldcg(reinterpret_cast<const uint4*>(token_addr(tok, g, (long long)row * g.W + w, c0 + v * 8))), f);
      if (pair) sm_unpack8(__ldcg(reinterpret_cast<const uint4*>(token_addr(tok, g, (long long)row * g.W + g.W - w, c0 + v * 8))), h);
    } else {
      for (int q = 0; q < 8; ++q) f[q] = h[q] = nanv;
    }
    if (pair) {
      for (int q = 0; q < 8; ++q) {
        xe[(w - 1) * g.Cb + v * 8 + q] = f[q] + h[q];
        xo[(w - 1) * g.Cb + v * 8 + q] = f[q] - h[q];
      }
    } else {
      float* dst = w == 0 ? x0 : xh;
      for (int q = 0; q < 8; ++q) dst[v * 8 + q] = f[q];
    }
  }
  __syncthreads();
  const int cp = tid % CP, kg = tid / CP;
  if (kg >= groups) return;
  const float inv = rsqrtf((float)g.W);
  const int ldy = g.nblk * g.Cb;
  const float2* xe2 = reinterpret_cast<const float2*>(xe);
  const float2* xo2 = reinterpret_cast<const float2*>(xo);
  const float2 a0 = reinterpret_cast<const float2*>(x0)[cp], ah = reinterpret_cast<const float2*>(xh)[cp];
  for (int pass = 0; pass < passes; ++pass) {
    const int k0 = (pass * groups + kg) * kRowNK;
    if (k0 >= g.KX) break;
    float re0[kRowNK], re1[kRowNK], im0[kRowNK], im1[kRowNK];
#pragma unroll
    for (int q = 0; q < kRowNK; ++q) re0[q] = re1[q] = im0[q] = im1[q] = 0.f;
    for (int wi = 0; wi < nfold; ++wi) {
      const float2 e = xe2[wi * CP + cp], o = xo2[wi * CP + cp];
      const float4* t4 = reinterpret_cast<const float4*>(tw2 + (size_t)wi * pad + k0);
#pragma unroll
      for (int q = 0; q < kRowNK / 2; ++q) {
        const float4 t = t4[q];
        re0[2 * q] += e.x * t.x;      re1[2 * q] += e.y * t.x;
        im0[2 * q] -= o.x * t.y;      im1[2 * q] -= o.y * t.y;
        re0[2 * q + 1] += e.x * t.z;  re1[2 * q + 1] += e.y * t.z;
        im0[2 * q + 1] -= o.x * t.w;  im1[2 * q + 1] -= o.y * t.w;
      }
    }
#pragma unroll
    for (int q = 0; q < kRowNK; ++q) {
      const int kx = k0 + q;
      if (kx < g.KX) {
        const float sg = (kx & 1) ? -1.f : 1.f;
        const float s = inv * ((kweight && kx > 0) ? 2.f : 1.f);
        float4 out;
        out.x = (re0[q] + a0.x + sg * ah.x) * s;  out.y = im0[q] * s;
        out.z = (re1[q] + a0.y + sg * ah.y) * s;  out.w = im1[q] * s;
        *reinterpret_cast<float4*>(Y + ((size_t)row * g.KX + kx) * ldy + j * g.Cb + 2 * cp) = out;
      }
    }
  }
}

__global__ void __launch_bounds__(512)
afno_rows_c2r_v2_kernel(const float2* __restrict__ X, TokenPtrs tok, AfGeom g, int kweight, PeerArgs peer, int signal,
                        unsigned int* counter, int groups, int passes, const __nv_bfloat16* __restrict__ add0,
                        const __nv_bfloat16* __restrict__ add1) {
  extern __shared__ float sm[];
  const int Wh = g.W >> 1, CP = g.Cb >> 1;
  const int pad = passes * groups * kRowNK;                       // >= W/2 + 1 positions w = 0 .. W/2
  float2* xs = reinterpret_cast<float2*>(sm);                     // [KX][Cb] spectrum, weighted
  float2* twT = xs + (size_t)g.KX * g.Cb;                         // [KX][pad]
  __nv_bfloat16* ys = reinterpret_cast<__nv_bfloat16*>(twT + (size_t)g.KX * pad);   // [W][Cb]
  const int row = blockIdx.x, j = blockIdx.y, tid = threadIdx.x, nt = blockDim.x;
  const int ldx = g.nblk * g.Cb;
  for (int i = tid; i < g.KX * pad; i += nt) {
    const int kx = i / pad, w = i % pad;
    float sn, cs;
    sincospif(2.f * ((kx * w) % g.W) / g.W, &sn, &cs);
    twT[i] = make_float2(cs, sn);
  }
  for (int i = tid; i < g.KX * g.Cb; i += nt) {
    const int kx = i / g.Cb, c = i % g.Cb;
    const float2 v = X[((size_t)row * g.KX + kx) * ldx + j * g.Cb + c];
    const float s = (kweight && kx > 0) ? 2.f : 1.f;
    xs[i] = make_float2(v.x * s, v.y * s);
  }
  __syncthreads();
  const int cp = tid % CP, wg = tid / CP;
  if (wg < groups) {
    const float inv = rsqrtf((float)g.W);
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    for (int pass = 0; pass < passes; ++pass) {
      const int w0 = (pass * groups + wg) * kRowNK;
      if (w0 > Wh) break;
      float A0[kRowNK], A1[kRowNK], B0[kRowNK], B1[kRowNK];
#pragma unroll
      for (int q = 0; q < kRowNK; ++q) A0[q] = A1[q] = B0[q] = B1[q] = 0.f;
      for (int kx = 0; kx < g.KX; ++kx) {
        const float4 xv = xs4[kx * CP + cp];                      // (re, im) of the two channels
        const float4* t4 = reinterpret_cast<const float4*>(twT + (size_t)kx * pad + w0);
#pragma unroll
        for (int q = 0; q < kRowNK / 2; ++q) {
          const float4 t = t4[q];
          A0[2 * q] += xv.x * t.x;      B0[2 * q] += xv.y * t.y;
          A1[2 * q] += xv.z * t.x;      B1[2 * q] += xv.w * t.y;
          A0[2 * q + 1] += xv.x * t.z;  B0[2 * q + 1] += xv.y * t.w;
          A1[2 * q + 1] += xv.z * t.z;  B1[2 * q + 1] += xv.w * t.w;
        }
      }
#pragma unroll
      for (int q = 0; q < kRowNK; ++q) {
        const int w = w0 + q;
        if (w <= Wh) {
          *reinterpret_cast<uint32_t*>(ys + w * g.Cb + 2 * cp) = pack_bf16x2((A0[q] - B0[q]) * inv, (A1[q] - B1[q]) * inv);
          if (w > 0 && w < Wh)
            *reinterpret_cast<uint32_t*>(ys + (g.W - w) * g.Cb + 2 * cp) = pack_bf16x2((A0[q] + B0[q]) * inv, (A1[q] + B1[q]) * inv);
        }
      }
    }
  }
  __syncthreads();
  const int c0 = (g.blk0 + j) * g.Cb;
  const int vec = g.Cb >> 3;
  for (int i = tid; i < g.W * vec; i += nt) {
    const int w = i / vec, v = i % vec;
    uint4 u = *reinterpret_cast<const uint4*>(ys + w * g.Cb + v * 8);
    if (add0) {
      // residual terms of the surrounding block (local [T, C] token layout), summed in fp32 and rounded once
      const long long at = ((long long)row * g.W + w) * g.C + c0 + v * 8;
      float f[8], a[8];
      sm_unpack8(u, f);
      sm_unpack8(*reinterpret_cast<const uint4*>(add0 + at), a);
#pragma unroll
      for (int q = 0; q < 8; ++q) f[q] += a[q];
      if (add1) {
        sm_unpack8(*reinterpret_cast<const uint4*>(add1 + at), a);
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] += a[q];
      }
      u = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
    }
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

// ---------------------------------------------------------------------- columns, split form (MLP on the tensor cores)
// The two-layer complex MLP is two real GEMMs on the [real | imag] expansion of the spectrum, so under bf16 compute it
// belongs on the tcgen05 GEMM kernel (the reference's einsums run in bf16 under autocast as well).  The two kernels below
// are the Fourier halves around those GEMMs.  E: bf16 [nblk][Mp][2 Cb] with row (b*KX + kx)*H + ky of a block's Mp
// (>= B*KX*H, the GEMM's padding) rows, columns [real | imag].
//   cols_dft : E = DFT_H(Y) (sign -1), optionally masked: entries whose counterpart in `mask` (same layout, the pre-shrink
//              MLP output of the forward) has magnitude <= lambda are zeroed (backward of the soft-shrink)
//   cols_idft: Yout = IDFT_H(softshrink_lambda(E)) (sign +1; lambda = 0 leaves E unchanged)
// ------------------------------------------------- columns, register-blocked form of the split (tensor-core MLP) stage
// [H][CH] complex data of a chunk of CH channels in shared memory (two buffers), H = H1 * H2.  A work item is a channel
// PAIR, one inner index and a block of kColNB outputs, so that a data vector read once (16 bytes: two complex values)
// meets kColNB twiddles (warp-uniform addresses) in 8 kColNB multiply-adds with 4 kColNB independent accumulators.
// Tables (sign folded in): w1[k1][n1] = e^{s 2 pi i n1 k1 / H1}, wm[k1][n2] = e^{s 2 pi i n2 k1 / H}, w2[k2][n2] = e^{s 2 pi i n2 k2 / H2}.
constexpr int kColNB = 5;

__device__ __forceinline__ void col_tables(float2* w1, float2* wm, float2* w2, int H1, int H2, float sign) {
  const int H = H1 * H2;
  for (int i = threadIdx.x; i < H1 * H1 + H + H2 * H2; i += blockDim.x) {
    float sn, cs;
    if (i < H1 * H1) {
      sincospif(2.f * (((i / H1) * (i % H1)) % H1) / H1, &sn, &cs);
      w1[i] = make_float2(cs, sign * sn);
    } else if (i < H1 * H1 + H) {
      const int t = i - H1 * H1;                                   // t = k1 * H2 + n2
      sincospif(2.f * (((t / H2) * (t % H2)) % H) / H, &sn, &cs);
      wm[t] = make_float2(cs, sign * sn);
    } else {
      const int t = i - H1 * H1 - H;
      sincospif(2.f * (((t / H2) * (t % H2)) % H2) / H2, &sn, &cs);
      w2[t] = make_float2(cs, sign * sn);
    }
  }
}

// a -> b -> a;  the caller synchronises before (a and the tables complete); a is complete on return
__device__ void col_dft_v2(float2* a, float2* b, const float2* w1, const float2* wm, const float2* w2, int H1, int H2, int CH) {
  const int CP = CH >> 1, tid = threadIdx.x, nt = blockDim.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  float4* b4 = reinterpret_cast<float4*>(b);
  const int nb1 = (H1 + kColNB - 1) / kColNB;
  for (int item = tid; item < nb1 * H2 * CP; item += nt) {
    const int cp = item % CP, r = item / CP, n2 = r % H2, k10 = (r / H2) * kColNB;
    float2 p[kColNB], q[kColNB];
#pragma unroll
    for (int u = 0; u < kColNB; ++u) p[u] = q[u] = make_float2(0.f, 0.f);
    for (int n1 = 0; n1 < H1; ++n1) {
      const float4 v = a4[(H2 * n1 + n2) * CP + cp];
#pragma unroll
      for (int u = 0; u < kColNB; ++u) {
        const float2 t = w1[min(k10 + u, H1 - 1) * H1 + n1];
        p[u].x += v.x * t.x - v.y * t.y;  p[u].y += v.x * t.y + v.y * t.x;
        q[u].x += v.z * t.x - v.w * t.y;  q[u].y += v.z * t.y + v.w * t.x;
      }
    }
#pragma unroll
    for (int u = 0; u < kColNB; ++u) {
      const int k1 = k10 + u;
      if (k1 < H1) {
        const float2 t = wm[k1 * H2 + n2];
        const float2 x = cmul(p[u], t), y = cmul(q[u], t);
        b4[(k1 * H2 + n2) * CP + cp] = make_float4(x.x, x.y, y.x, y.y);
      }
    }
  }
  __syncthreads();
  const float inv = rsqrtf((float)(H1 * H2));
  const float4* bb4 = reinterpret_cast<const float4*>(b);
  float4* o4 = reinterpret_cast<float4*>(a);
  const int nb2 = (H2 + kColNB - 1) / kColNB;
  for (int item = tid; item < nb2 * H1 * CP; item += nt) {
    const int cp = item % CP, r = item / CP, k1 = r % H1, k20 = (r / H1) * kColNB;
    float2 p[kColNB], q[kColNB];
#pragma unroll
    for (int u = 0; u < kColNB; ++u) p[u] = q[u] = make_float2(0.f, 0.f);
    for (int n2 = 0; n2 < H2; ++n2) {
      const float4 v = bb4[(k1 * H2 + n2) * CP + cp];
#pragma unroll
      for (int u = 0; u < kColNB; ++u) {
        const float2 t = w2[min(k20 + u, H2 - 1) * H2 + n2];
        p[u].x += v.x * t.x - v.y * t.y;  p[u].y += v.x * t.y + v.y * t.x;
        q[u].x += v.z * t.x - v.w * t.y;  q[u].y += v.z * t.y + v.w * t.x;
      }
    }
#pragma unroll
    for (int u = 0; u < kColNB; ++u) {
      const int k2 = k20 + u;
      if (k2 < H2) o4[(k1 + H1 * k2) * CP + cp] = make_float4(p[u].x * inv, p[u].y * inv, q[u].x * inv, q[u].y * inv);
    }
  }
  __syncthreads();
}

struct ColSmem { float2 *a, *b, *w1, *wm, *w2; };
__device__ __forceinline__ ColSmem col_smem(float* sm, int H, int H1, int H2, int CH) {
  ColSmem c;
  c.a = reinterpret_cast<float2*>(sm);
  c.b = c.a + (size_t)H * CH;
  c.w1 = c.b + (size_t)H * CH;
  c.wm = c.w1 + H1 * H1;
  c.w2 = c.wm + H;
  return c;
}

// blockIdx.y = owned block * chunks + chunk;  CH = Cb / chunks channels per CTA
__global__ void __launch_bounds__(256)
afno_cols_dft_v2_kernel(const float2* __restrict__ Y, __nv_bfloat16* __restrict__ E, const __nv_bfloat16* __restrict__ mask, AfGeom g,
                        float lambda, int chunks, int Mp) {
  extern __shared__ float sm[];
  const int CH = g.Cb / chunks;
  const ColSmem s = col_smem(sm, g.H, g.H1, g.H2, CH);
  const int bk = blockIdx.x, j = blockIdx.y / chunks, coff = (blockIdx.y % chunks) * CH, tid = threadIdx.x, nt = blockDim.x;
  const int bb = bk / g.KX, kx = bk % g.KX;
  const int ld = g.nblk * g.Cb;
  col_tables(s.w1, s.wm, s.w2, g.H1, g.H2, -1.f);
  for (int i = tid; i < g.H * CH; i += nt) {
    const int h = i / CH, c = i % CH;
    s.a[i] = Y[((size_t)(bb * g.H + h) * g.KX + kx) * ld + j * g.Cb + coff + c];
  }
  __syncthreads();
  col_dft_v2(s.a, s.b, s.w1, s.wm, s.w2, g.H1, g.H2, CH);
  const size_t base = ((size_t)j * Mp + (size_t)bk * g.H) * (2 * g.Cb) + coff;
  const int CP = CH >> 1;
  for (int i = tid; i < g.H * CP; i += nt) {
    const int ky = i / CP, cp = i % CP;
    float4 v = reinterpret_cast<const float4*>(s.a)[i];           // (re, im) of channels 2 cp, 2 cp + 1
    const size_t o = base + (size_t)ky * 2 * g.Cb + 2 * cp;
    if (mask) {
      const float2 mr = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(mask + o));
      const float2 mi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(mask + o + g.Cb));
      if (fabsf(mr.x) <= lambda) v.x = 0.f;
      if (fabsf(mi.x) <= lambda) v.y = 0.f;
      if (fabsf(mr.y) <= lambda) v.z = 0.f;
      if (fabsf(mi.y) <= lambda) v.w = 0.f;
    }
    *reinterpret_cast<uint32_t*>(E + o) = pack_bf16x2(v.x, v.z);
    *reinterpret_cast<uint32_t*>(E + o + g.Cb) = pack_bf16x2(v.y, v.w);
  }
}

__global__ void __launch_bounds__(256)
afno_cols_idft_v2_kernel(const __nv_bfloat16* __restrict__ E, float2* __restrict__ Yout, AfGeom g, float lambda, int chunks,
                         int Mp) {
  extern __shared__ float sm[];
  const int CH = g.Cb / chunks;
  const ColSmem s = col_smem(sm, g.H, g.H1, g.H2, CH);
  const int bk = blockIdx.x, j = blockIdx.y / chunks, coff = (blockIdx.y % chunks) * CH, tid = threadIdx.x, nt = blockDim.x;
  const int bb = bk / g.KX, kx = bk % g.KX;
  const int ld = g.nblk * g.Cb;
  col_tables(s.w1, s.wm, s.w2, g.H1, g.H2, +1.f);
  const size_t base = ((size_t)j * Mp + (size_t)bk * g.H) * (2 * g.Cb) + coff;
  const int CP = CH >> 1;
  for (int i = tid; i < g.H * CP; i += nt) {
    const int ky = i / CP, cp = i % CP;
    const size_t o = base + (size_t)ky * 2 * g.Cb + 2 * cp;
    float2 re = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(E + o));
    float2 im = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(E + o + g.Cb));
    if (lambda > 0.f) {
      re.x = softshrink_f(re.x, lambda); re.y = softshrink_f(re.y, lambda);
      im.x = softshrink_f(im.x, lambda); im.y = softshrink_f(im.y, lambda);
    }
    reinterpret_cast<float4*>(s.a)[i] = make_float4(re.x, im.x, re.y, im.y);
  }
  __syncthreads();
  col_dft_v2(s.a, s.b, s.w1, s.wm, s.w2, g.H1, g.H2, CH);
  for (int i = tid; i < g.H * CH; i += nt) {
    const int h = i / CH, c = i % CH;
    Yout[((size_t)(bb * g.H + h) * g.KX + kx) * ld + j * g.Cb + coff + c] = s.a[i];
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
  pnm::PeerArgs p{};
  if (wait) p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  if (g.W % 2 == 0 && g.W >= 4) {
    const pnm::RowPlan rp = pnm::row_plan(g.KX, g.Cb);
    const size_t smem2 = sizeof(float) * (2 * (size_t)(g.W / 2) * g.Cb + 2 * (size_t)(g.W / 2 - 1) * rp.pad);
    if (smem2 <= 220 * 1024) {
      static unsigned long long mask2 = 0;
      if (int rc = pnm::af_smem_attr(pnm::afno_rows_r2c_v2_kernel, smem2, mask2)) return rc;
      pnm::afno_rows_r2c_v2_kernel<<<dim3(g.B * g.H, g.nblk), rp.threads, smem2, (cudaStream_t)stream>>>(
          pnm::make_tok(tokens), (float2*)Y, g, kweight, p, wait, err, rp.groups, rp.passes);
      return cudaGetLastError() == cudaSuccess ? 0 : -3;
    }
  }
  const size_t smem = sizeof(float) * ((size_t)g.W * g.Cb + 2 * g.W);
  static unsigned long long mask = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_rows_r2c_kernel, smem, mask)) return rc;
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
  pnm::PeerArgs p{};
  if (signal) p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, 1.0, epoch_base);
  if (g.W % 2 == 0 && g.W >= 4) {
    const pnm::RowPlan rp = pnm::row_plan(g.W / 2 + 1, g.Cb);
    const size_t smem2 = sizeof(float2) * ((size_t)g.KX * g.Cb + (size_t)g.KX * rp.pad) + sizeof(__nv_bfloat16) * (size_t)g.W * g.Cb;
    if (smem2 <= 220 * 1024) {
      static unsigned long long mask2 = 0;
      if (int rc = pnm::af_smem_attr(pnm::afno_rows_c2r_v2_kernel, smem2, mask2)) return rc;
      pnm::afno_rows_c2r_v2_kernel<<<dim3(g.B * g.H, g.nblk), rp.threads, smem2, (cudaStream_t)stream>>>(
          (const float2*)X, pnm::make_tok(tokens), g, kweight, p, signal, (unsigned int*)counter, rp.groups, rp.passes, nullptr,
          nullptr);
      return cudaGetLastError() == cudaSuccess ? 0 : -3;
    }
  }
  const size_t smem = sizeof(float2) * ((size_t)g.KX * g.Cb + g.W) + sizeof(__nv_bfloat16) * (size_t)g.W * g.Cb;
  static unsigned long long mask = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_rows_c2r_kernel, smem, mask)) return rc;
  pnm::afno_rows_c2r_kernel<<<dim3(g.B * g.H, g.nblk), 2 * g.Cb, smem, (cudaStream_t)stream>>>((const float2*)X, pnm::make_tok(tokens),
                                                                                              g, kweight, p, signal,
                                                                                              (unsigned int*)counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Single-GPU form of pnm_afno_rows_c2r that also adds up to two residual tensors (add0, add1: [T, C] bf16, add1 may be
// null) to the transformed tokens before the store.  -2 when the shape needs the fallback row kernel (no addends there).
int pnm_afno_rows_c2r_add(const void* X, void* out, const void* add0, const void* add1, const int* geom, long long Tp, int kweight,
                          void* stream) {
  pnm::AfGeom g{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], Tp, geom[8], geom[9]};
  if (pnm::af_check(g) || !out || !add0) return -2;
  if (g.W % 2 || g.W < 4) return -2;
  const pnm::RowPlan rp = pnm::row_plan(g.W / 2 + 1, g.Cb);
  const size_t smem2 = sizeof(float2) * ((size_t)g.KX * g.Cb + (size_t)g.KX * rp.pad) + sizeof(__nv_bfloat16) * (size_t)g.W * g.Cb;
  if (smem2 > 220 * 1024) return -2;
  static unsigned long long mask2 = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_rows_c2r_v2_kernel, smem2, mask2)) return rc;
  const void* ptrs[8] = {out, out, out, out, out, out, out, out};
  pnm::afno_rows_c2r_v2_kernel<<<dim3(g.B * g.H, g.nblk), rp.threads, smem2, (cudaStream_t)stream>>>(
      (const float2*)X, pnm::make_tok(ptrs), g, kweight, pnm::PeerArgs{}, 0, nullptr, rp.groups, rp.passes,
      (const __nv_bfloat16*)add0, (const __nv_bfloat16*)add1);
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

// Split form of the column stage (see afno_cols_dft_v2_kernel): E bf16 [nblk, Mp, 2*Cb]; mask optional (same layout).
int pnm_afno_cols_dft(const void* Y, void* E, const void* mask, const int* geom, int Mp, float lambda, void* stream) {
  pnm::AfGeom g{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], 1, geom[8], geom[9]};
  if (pnm::af_check(g) || Mp < g.B * g.KX * g.H) return -2;
  const int chunks = (g.Cb % 16 == 0 && g.Cb >= 64) ? 2 : 1;
  const size_t smem = sizeof(float2) * (2 * (size_t)g.H * (g.Cb / chunks) + g.H1 * g.H1 + g.H + g.H2 * g.H2);
  static unsigned long long mask_bits = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_cols_dft_v2_kernel, smem, mask_bits)) return rc;
  pnm::afno_cols_dft_v2_kernel<<<dim3(g.B * g.KX, g.nblk * chunks), 256, smem, (cudaStream_t)stream>>>(
      (const float2*)Y, (__nv_bfloat16*)E, (const __nv_bfloat16*)mask, g, lambda, chunks, Mp);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int pnm_afno_cols_idft(const void* E, void* Yout, const int* geom, int Mp, float lambda, void* stream) {
  pnm::AfGeom g{geom[0], geom[1], geom[2], geom[3], geom[4], geom[5], geom[6], geom[7], 1, geom[8], geom[9]};
  if (pnm::af_check(g) || Mp < g.B * g.KX * g.H) return -2;
  const int chunks = (g.Cb % 16 == 0 && g.Cb >= 64) ? 2 : 1;
  const size_t smem = sizeof(float2) * (2 * (size_t)g.H * (g.Cb / chunks) + g.H1 * g.H1 + g.H + g.H2 * g.H2);
  static unsigned long long mask_bits = 0;
  if (int rc = pnm::af_smem_attr(pnm::afno_cols_idft_v2_kernel, smem, mask_bits)) return rc;
  pnm::afno_cols_idft_v2_kernel<<<dim3(g.B * g.KX, g.nblk * chunks), 256, smem, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)E, (float2*)Yout, g, lambda, chunks, Mp);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
