// The small (parameter- and slice-token-sized) algebra of the fused Transolver physics attention, forward and backward,
// as four kernels.  The large passes over the N points are tcgen05 GEMMs (gemm_tn / gemm_nt); what is left per block is
// a chain of ~130 tiny tensor operations on matrices of at most 512 x 512 values, whose launch overhead does not shrink
// when the points are sharded.  Notation: H heads, S = 64 slices, D = head width, inner = H * D, C = channels of x.
//
//   pa_prepare_fwd   Wc = blockdiag_H(Ws) Wx (bf16), bc, 1 / clamp(T), bf16 copy of Wfx, Wback = [Wc^T | Wfx^T] (bf16)
//   pa_tokens_fwd    slice tokens (sum over ranks by peer loads in the prologue) -> normalise -> q k v -> 64 x 64
//                    attention per head -> Wcomb = Wo blockdiag(out_tokens)^T (bf16 + fp32)
//   pa_tokens_bwd    dWcomb (sum over ranks in the prologue) -> d out_tokens, dWo -> attention backward -> d tokens,
//                    dWqkv -> the operands of the point-sized backward GEMMs: Bcat = [Wcomb^T | blockdiag(d_tok)],
//                    BdT = blockdiag(d_tok)^T (bf16), d_norm
//   pa_prepare_bwd   dWx, dbx, dWs, dbs, dT from dWc, dbc and the per-head temperature sums
//
// Cross-rank sums: the producers (gemm_nt) write into a region of this rank's symmetric buffer, a signal kernel raises
// the flags, and the token kernels add the P copies with direct peer loads after a bounded wait -- there is no
// stand-alone all-reduce.  With world == 1 the source is an ordinary local buffer and no flag is touched.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"
#include "pnm_internal.h"

namespace pnm {

constexpr int kPaS = 64;
constexpr int kPaMaxD = 64;
constexpr int kPaTokenThreads = 1024;   // the token kernels are latency-bound chains: 32 warps hide the shared-memory latency

struct PaSrc {
  const float* p[kPeerMaxRanks];  // per rank: base of the partial-sum matrix (peer-mapped for r != rank)
  int world;
  int use_flags;                  // wait for the ranks' "small" flags of the call before reading
};

__device__ __forceinline__ float pa_sum(const PaSrc& s, long long i) {
  float a = 0.f;
  for (int r = 0; r < s.world; ++r) a += __ldcg(s.p[r] + i);
  return a;
}

__device__ __forceinline__ bool pa_wait(const PaSrc& s, const PeerArgs& peer, int* err, int* sh_ok) {
  if (!s.use_flags) return true;
  return peer_small_wait(peer, peer_epoch(peer), err, sh_ok);
}

// grid H*S + inner, 256 threads
__global__ void __launch_bounds__(256)
pa_prepare_fwd_kernel(const float* __restrict__ Wx, const float* __restrict__ bx, const float* __restrict__ Wfx,
                      const float* __restrict__ Ws, const float* __restrict__ bs, const float* __restrict__ temp,
                      __nv_bfloat16* __restrict__ Wc, float* __restrict__ bc, float* __restrict__ inv_t,
                      __nv_bfloat16* __restrict__ Wfx16, __nv_bfloat16* __restrict__ Wback, int H, int D, int C) {
  __shared__ float ws[kPaMaxD];
  const int HS = H * kPaS, inner = H * D, ldb = HS + inner;
  const int r = blockIdx.x;
  if (r < HS) {
    const int h = r / kPaS, s = r % kPaS;
    if (threadIdx.x < D) ws[threadIdx.x] = Ws[s * D + threadIdx.x];
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float acc = 0.f;
      for (int d = 0; d < D; ++d) acc += ws[d] * Wx[(size_t)(h * D + d) * C + c];
      const __nv_bfloat16 v = __float2bfloat16(acc);
      Wc[(size_t)r * C + c] = v;
      Wback[(size_t)c * ldb + r] = v;
    }
    if (threadIdx.x == 0) {
      float acc = bs[s];
      for (int d = 0; d < D; ++d) acc += ws[d] * bx[h * D + d];
      bc[r] = acc;
      inv_t[r] = 1.f / fminf(fmaxf(temp[h], 0.5f), 5.f);
    }
  } else {
    const int j = r - HS;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      const __nv_bfloat16 v = __float2bfloat16(Wfx[(size_t)j * C + c]);
      Wfx16[(size_t)j * C + c] = v;
      Wback[(size_t)c * ldb + HS + j] = v;
    }
  }
}

struct PaSaved {        // per block, fp32, all [H][S][...]
  float* token;         // [H][S][D]
  float* normp;         // [H][S]      norm + 0.01
  float* q; float* k; float* v;   // [H][S][D]
  float* prob;          // [H][S][S]
  float* out;           // [H][S][D]
  float* wcomb;         // [Cout][H*S]
};

// grid H, kPaTokenThreads threads, dynamic shared memory (see pa_fwd_smem).  One CTA per head: the work per head is a
// chain of dependent 64 x 64 x D products, so the only parallelism to add inside a head is more warps per phase.
__global__ void __launch_bounds__(kPaTokenThreads)
pa_tokens_fwd_kernel(PaSrc src, long long norm_off, int ld_tok, const float* __restrict__ Wqkv, const float* __restrict__ Wo,
                     __nv_bfloat16* __restrict__ wcomb16, PaSaved sv, int H, int D, int Cout, float scale, PeerArgs peer, int* err) {
  extern __shared__ float sm[];
  __shared__ int sh_ok;
  const int S = kPaS, P1 = D + 1;
  float* tok = sm;                 // [S][D+1]
  float* q = tok + S * P1;
  float* k = q + S * P1;
  float* v = k + S * P1;
  float* o = v + S * P1;
  float* pr = o + S * P1;          // [S][S+1]
  float* wq = pr + S * (S + 1);    // [3D][D+1]  padded rows: the q k v product reads one row per lane
  float* wo_s = wq + 3 * D * P1;   // [Cout][D+1]  this head's columns of Wo
  const int h = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const int HS = H * S, inner = H * D;
  const bool ok = pa_wait(src, peer, err, &sh_ok);
  const float nanv = __int_as_float(0x7fc00000);
  for (int i = tid; i < 3 * D * D; i += nt) wq[(i / D) * P1 + (i % D)] = Wqkv[i];
  for (int i = tid; i < Cout * D; i += nt) wo_s[(i / D) * P1 + (i % D)] = Wo[(size_t)(i / D) * inner + h * D + (i % D)];
  for (int i = tid; i < S * D; i += nt) {
    const int s = i / D, d = i % D;
    const float nrm = ok ? pa_sum(src, norm_off + h * S + s) + 1e-2f : nanv;
    const float t = ok ? pa_sum(src, (long long)(h * S + s) * ld_tok + h * D + d) : nanv;
    const float tk = t / nrm;
    tok[s * P1 + d] = tk;
    sv.token[(size_t)(h * S + s) * D + d] = tk;
    if (d == 0) sv.normp[h * S + s] = nrm;
  }
  __syncthreads();
  for (int i = tid; i < S * 3 * D; i += nt) {
    const int s = i / (3 * D), j = i % (3 * D);
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc += tok[s * P1 + d] * wq[j * P1 + d];
    float* dst = j < D ? q : (j < 2 * D ? k : v);
    float* gsv = j < D ? sv.q : (j < 2 * D ? sv.k : sv.v);
    dst[s * P1 + (j % D)] = acc;
    gsv[(size_t)(h * S + s) * D + (j % D)] = acc;
  }
  __syncthreads();
  for (int i = tid; i < S * S; i += nt) {
    const int s = i / S, t = i % S;
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc += q[s * P1 + d] * k[t * P1 + d];
    pr[s * (S + 1) + t] = acc * scale;
  }
  __syncthreads();
  {  // softmax over t: one warp per row, two columns per lane
    const int warp = tid >> 5, lane = tid & 31, nw = nt >> 5;
    for (int s = warp; s < S; s += nw) {
      float a = pr[s * (S + 1) + lane], b = pr[s * (S + 1) + lane + 32];
      float m = fmaxf(a, b);
      for (int x = 16; x > 0; x >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, x));
      a = __expf(a - m); b = __expf(b - m);
      float z = a + b;
      for (int x = 16; x > 0; x >>= 1) z += __shfl_xor_sync(0xffffffffu, z, x);
      const float inv = 1.f / z;
      pr[s * (S + 1) + lane] = a * inv;
      pr[s * (S + 1) + lane + 32] = b * inv;
      sv.prob[(size_t)(h * S + s) * S + lane] = a * inv;
      sv.prob[(size_t)(h * S + s) * S + lane + 32] = b * inv;
    }
  }
  __syncthreads();
  for (int i = tid; i < S * D; i += nt) {
    const int s = i / D, d = i % D;
    float acc = 0.f;
    for (int t = 0; t < S; ++t) acc += pr[s * (S + 1) + t] * v[t * P1 + d];
    o[s * P1 + d] = acc;
    sv.out[(size_t)(h * S + s) * D + d] = acc;
  }
  __syncthreads();
  for (int i = tid; i < Cout * S; i += nt) {
    const int c = i / S, s = i % S;
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc += wo_s[c * P1 + d] * o[s * P1 + d];
    wcomb16[(size_t)c * HS + h * S + s] = __float2bfloat16(acc);
    sv.wcomb[(size_t)c * HS + h * S + s] = acc;
  }
}

// grid H, kPaTokenThreads threads, dynamic shared memory
__global__ void __launch_bounds__(kPaTokenThreads)
pa_tokens_bwd_kernel(PaSrc src, const float* __restrict__ Wqkv, const float* __restrict__ Wo, PaSaved sv,
                     float* __restrict__ dWo, float* __restrict__ dWqkv, float* __restrict__ d_norm,
                     __nv_bfloat16* __restrict__ Bcat, __nv_bfloat16* __restrict__ BdT, int H, int D, int Cout, float scale,
                     float share, PeerArgs peer, int* err) {
  extern __shared__ float sm[];
  __shared__ int sh_ok;
  const int S = kPaS, P1 = D + 1, SP = S + 1;
  float* dwc = sm;                 // [Cout][S+1]   this head's columns of dWcomb
  float* dout = dwc + Cout * SP;   // [S][D+1]
  float* q = dout + S * P1;
  float* k = q + S * P1;
  float* v = k + S * P1;
  float* tok = v + S * P1;
  float* dq = tok + S * P1;
  float* dk = dq + S * P1;
  float* dv = dk + S * P1;
  float* pr = dv + S * P1;         // [S][S+1]
  float* ds = pr + S * SP;         // [S][S+1]
  float* wq = ds + S * SP;         // [3D][D]
  float* rowdot = wq + 3 * D * D;  // [S]
  float* wo_s = rowdot + S;        // [Cout][D+1]  this head's columns of Wo
  const int h = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
  const int HS = H * S, inner = H * D;
  const bool ok = pa_wait(src, peer, err, &sh_ok);
  const float nanv = __int_as_float(0x7fc00000);
  for (int i = tid; i < Cout * S; i += nt) {
    const int c = i / S, s = i % S;
    dwc[c * SP + s] = ok ? pa_sum(src, (long long)c * HS + h * S + s) : nanv;
  }
  for (int i = tid; i < 3 * D * D; i += nt) wq[i] = Wqkv[i];
  for (int i = tid; i < Cout * D; i += nt) wo_s[(i / D) * P1 + (i % D)] = Wo[(size_t)(i / D) * inner + h * D + (i % D)];
  for (int i = tid; i < S * D; i += nt) {
    const int s = i / D, d = i % D;
    const size_t g = (size_t)(h * S + s) * D + d;
    q[s * P1 + d] = sv.q[g]; k[s * P1 + d] = sv.k[g]; v[s * P1 + d] = sv.v[g]; tok[s * P1 + d] = sv.token[g];
    dq[s * P1 + d] = sv.out[g];          // dq holds the attention output until the attention backward overwrites it
  }
  for (int i = tid; i < S * S; i += nt) pr[(i / S) * SP + (i % S)] = sv.prob[(size_t)h * S * S + i];
  __syncthreads();
  // d out_tokens[s][d] = sum_c dWcomb[c][s] Wo[c][h D + d];  dWo[c][h D + d] = sum_s dWcomb[c][s] out[s][d]
  for (int i = tid; i < S * D; i += nt) {
    const int s = i / D, d = i % D;
    float acc = 0.f;
    for (int c = 0; c < Cout; ++c) acc += dwc[c * SP + s] * wo_s[c * P1 + d];
    dout[s * P1 + d] = acc;
  }
  for (int i = tid; i < Cout * D; i += nt) {
    const int c = i / D, d = i % D;
    float acc = 0.f;
    for (int s = 0; s < S; ++s) acc += dwc[c * SP + s] * dq[s * P1 + d];
    dWo[(size_t)c * inner + h * D + d] = acc * share;
  }
  __syncthreads();
  // dWcomb is consumed: its buffer now stages this head's Wcomb^T tile for the coalesced Bcat rows written at the end
  for (int i = tid; i < Cout * S; i += nt) dwc[(i / S) * SP + (i % S)] = sv.wcomb[(size_t)(i / S) * HS + h * S + (i % S)];
  // dP = dout v^T ; dv = P^T dout
  for (int i = tid; i < S * S; i += nt) {
    const int s = i / S, t = i % S;
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc += dout[s * P1 + d] * v[t * P1 + d];
    ds[s * SP + t] = acc;
  }
  for (int i = tid; i < S * D; i += nt) {
    const int t = i / D, d = i % D;
    float acc = 0.f;
    for (int s = 0; s < S; ++s) acc += pr[s * SP + t] * dout[s * P1 + d];
    dv[t * P1 + d] = acc;
  }
  __syncthreads();
  if (tid < S) {
    float acc = 0.f;
    for (int t = 0; t < S; ++t) acc += ds[tid * SP + t] * pr[tid * SP + t];
    rowdot[tid] = acc;
  }
  __syncthreads();
  for (int i = tid; i < S * S; i += nt) {
    const int s = i / S, t = i % S;
    ds[s * SP + t] = pr[s * SP + t] * (ds[s * SP + t] - rowdot[s]) * scale;
  }
  __syncthreads();
  for (int i = tid; i < S * D; i += nt) {
    const int s = i / D, d = i % D;
    float a = 0.f, b = 0.f;
    for (int t = 0; t < S; ++t) { a += ds[s * SP + t] * k[t * P1 + d]; b += ds[t * SP + s] * q[t * P1 + d]; }
    dq[s * P1 + d] = a;   // dq[s] = sum_t dS[s][t] k[t]
    dk[s * P1 + d] = b;   // dk[s] = sum_t dS[t][s] q[t]
  }
  __syncthreads();
  // dWqkv[j][d] += share * sum_s dqkv[s][j] token[s][d]
  for (int i = tid; i < 3 * D * D; i += nt) {
    const int j = i / D, d = i % D;
    const float* g = j < D ? dq : (j < 2 * D ? dk : dv);
    const int jj = j % D;
    float acc = 0.f;
    for (int s = 0; s < S; ++s) acc += g[s * P1 + jj] * tok[s * P1 + d];
    atomicAdd(dWqkv + i, acc * share);
  }
  // d token[s][d] = sum_j dqkv[s][j] Wqkv[j][d]  (reuses dout as storage)
  __syncthreads();
  for (int i = tid; i < S * D; i += nt) {
    const int s = i / D, d = i % D;
    float acc = 0.f;
    for (int j = 0; j < D; ++j)
      acc += dq[s * P1 + j] * wq[j * D + d] + dk[s * P1 + j] * wq[(D + j) * D + d] + dv[s * P1 + j] * wq[(2 * D + j) * D + d];
    dout[s * P1 + d] = acc;
  }
  __syncthreads();
  if (tid < S) {
    const float np = sv.normp[h * S + tid];
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc += dout[tid * P1 + d] * tok[tid * P1 + d];
    d_norm[h * S + tid] = -acc / np;
    rowdot[tid] = 1.f / np;
  }
  __syncthreads();
  // Bcat rows h S + s: [Wcomb^T (Cout) | zeros ... d_tok[s][:] in block h ... zeros] ; BdT rows h D + d: d_tok[:, d] in block h
  const int ldc = Cout + inner;
  for (int i = tid; i < S * ldc; i += nt) {
    const int s = i / ldc, col = i % ldc;
    float val;
    if (col < Cout) val = dwc[col * SP + s];
    else {
      const int jd = col - Cout;
      val = (jd / D == h) ? dout[s * P1 + (jd % D)] * rowdot[s] : 0.f;
    }
    Bcat[(size_t)(h * S + s) * ldc + col] = __float2bfloat16(val);
  }
  for (int i = tid; i < D * HS; i += nt) {
    const int d = i / HS, col = i % HS;
    const int s = col % S;
    const float val = (col / S == h) ? dout[s * P1 + d] * rowdot[s] : 0.f;
    BdT[(size_t)(h * D + d) * HS + col] = __float2bfloat16(val);
  }
}

// grid inner + S * D / 8 + 1, 256 threads
__global__ void __launch_bounds__(256)
pa_prepare_bwd_kernel(const float* __restrict__ dWc, const float* __restrict__ dbc, const float* __restrict__ grp,
                      const float* __restrict__ Wx, const float* __restrict__ bx, const float* __restrict__ Ws,
                      const float* __restrict__ temp, float* __restrict__ dWx, float* __restrict__ dbx,
                      float* __restrict__ dWs, float* __restrict__ dbs, float* __restrict__ dtemp, int H, int D, int C) {
  const int S = kPaS, inner = H * D;
  const int b = blockIdx.x, tid = threadIdx.x;
  if (b < inner) {
    const int h = b / D, d = b % D;
    for (int c = tid; c < C; c += blockDim.x) {
      float acc = 0.f;
      for (int s = 0; s < S; ++s) acc += Ws[s * D + d] * dWc[(size_t)(h * S + s) * C + c];
      dWx[(size_t)b * C + c] = acc;
    }
    if (tid == 0) {
      float acc = 0.f;
      for (int s = 0; s < S; ++s) acc += Ws[s * D + d] * dbc[h * S + s];
      dbx[b] = acc;
    }
  } else if (b < inner + (S * D) / 8) {
    // dWs[s][d] = sum_h ( sum_c dWc[h S + s][c] Wx[h D + d][c] + dbc[h S + s] bx[h D + d] ): one warp per (s, d), lanes over c
    const int warp = tid >> 5, lane = tid & 31;
    const int e = (b - inner) * 8 + warp;
    const int s = e / D, d = e % D;
    float acc = 0.f;
    for (int h = 0; h < H; ++h) {
      const float* a = dWc + (size_t)(h * S + s) * C;
      const float* w = Wx + (size_t)(h * D + d) * C;
      for (int c = lane; c < C; c += 32) acc += a[c] * w[c];
    }
    for (int x = 16; x > 0; x >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, x);
    if (lane == 0) {
      float t = acc, bsum = 0.f;
      for (int h = 0; h < H; ++h) {
        t += dbc[h * S + s] * bx[h * D + d];
        bsum += dbc[h * S + s];
      }
      dWs[s * D + d] = t;
      if (d == 0) dbs[s] = bsum;
    }
  } else {
    for (int h = tid; h < H; h += blockDim.x) {
      const float T = temp[h];
      dtemp[h] = (T > 0.5f && T < 5.f) ? -grp[h] / T : 0.f;
    }
  }
}

static size_t pa_fwd_smem(int D, int Cout) {
  return sizeof(float) * (5 * kPaS * (D + 1) + kPaS * (kPaS + 1) + 3 * D * (D + 1) + (size_t)Cout * (D + 1));
}
static size_t pa_bwd_smem(int D, int Cout) {
  return sizeof(float) * ((size_t)Cout * (kPaS + 1) + 9 * kPaS * (D + 1) + 2 * kPaS * (kPaS + 1) + 3 * D * D + kPaS +
                          (size_t)Cout * (D + 1));
}

static PaSrc make_src(const void* const* srcs, int world, int use_flags) {
  PaSrc s;
  for (int r = 0; r < kPeerMaxRanks; ++r) s.p[r] = r < world ? reinterpret_cast<const float*>(srcs[r]) : nullptr;
  s.world = world;
  s.use_flags = use_flags;
  return s;
}

static PaSaved make_saved(void* const* p) {
  PaSaved s;
  s.token = (float*)p[0]; s.normp = (float*)p[1]; s.q = (float*)p[2]; s.k = (float*)p[3]; s.v = (float*)p[4];
  s.prob = (float*)p[5]; s.out = (float*)p[6]; s.wcomb = (float*)p[7];
  return s;
}

}  // namespace pnm

extern "C" {

int pnm_pa_prepare_fwd(const float* Wx, const float* bx, const float* Wfx, const float* Ws, const float* bs, const float* temp,
                       void* Wc16, float* bc, float* inv_t, void* Wfx16, void* Wback16, int H, int D, int C, void* stream) {
  if (H <= 0 || D <= 0 || D > pnm::kPaMaxD || C <= 0) return -2;
  pnm::pa_prepare_fwd_kernel<<<H * pnm::kPaS + H * D, 256, 0, (cudaStream_t)stream>>>(
      Wx, bx, Wfx, Ws, bs, temp, (__nv_bfloat16*)Wc16, bc, inv_t, (__nv_bfloat16*)Wfx16, (__nv_bfloat16*)Wback16, H, D, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// srcs: host array of `world` pointers to the [H*S, ld_tok] token-sum matrices (own first ... in rank order), whose
// element norm_off + h*S + s holds the slice norms.  saved: host array of 8 device pointers (token, normp, q, k, v,
// prob, out, wcomb).  use_flags != 0: wait for the peers' flags of call `epoch` (peer arguments as in pnm_peer_allreduce).
int pnm_pa_tokens_fwd(const void* const* srcs, int world, int use_flags, long long norm_off, int ld_tok, const float* Wqkv,
                      const float* Wo, void* wcomb16, void* const* saved, int H, int D, int Cout, float scale,
                      const void* const* bases, int rank, unsigned int epoch, long long capacity_floats, double budget_s,
                      const void* epoch_base, void* stream) {
  if (H <= 0 || D <= 0 || D > pnm::kPaMaxD || Cout <= 0 || world < 1 || world > pnm::kPeerMaxRanks) return -2;
  int* err = pnm::error_word_ptr();
  if (!err) return -1;
  const size_t smem = pnm::pa_fwd_smem(D, Cout);
  static unsigned long long mask = 0;
  if (pnm::first_use_on_device(mask) &&
      cudaFuncSetAttribute(pnm::pa_tokens_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
    return -4;
  if (smem > 160 * 1024) return -2;
  pnm::PeerArgs p{};
  if (use_flags) p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  pnm::pa_tokens_fwd_kernel<<<H, pnm::kPaTokenThreads, smem, (cudaStream_t)stream>>>(pnm::make_src(srcs, world, use_flags), norm_off, ld_tok, Wqkv,
                                                                   Wo, (__nv_bfloat16*)wcomb16, pnm::make_saved(saved), H, D,
                                                                   Cout, scale, p, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// srcs: per rank the [Cout, H*S] matrix dWcomb (partial sums).  dWqkv must be zero on entry (accumulated with atomics).
int pnm_pa_tokens_bwd(const void* const* srcs, int world, int use_flags, const float* Wqkv, const float* Wo, void* const* saved,
                      float* dWo, float* dWqkv, float* d_norm, void* Bcat16, void* BdT16, int H, int D, int Cout, float scale,
                      float share, const void* const* bases, int rank, unsigned int epoch, long long capacity_floats,
                      double budget_s, const void* epoch_base, void* stream) {
  if (H <= 0 || D <= 0 || D > pnm::kPaMaxD || Cout <= 0 || world < 1 || world > pnm::kPeerMaxRanks) return -2;
  int* err = pnm::error_word_ptr();
  if (!err) return -1;
  const size_t smem = pnm::pa_bwd_smem(D, Cout);
  if (smem > 226 * 1024) return -2;
  static unsigned long long mask = 0;
  if (pnm::first_use_on_device(mask) &&
      cudaFuncSetAttribute(pnm::pa_tokens_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess)
    return -4;
  pnm::PeerArgs p{};
  if (use_flags) p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  pnm::pa_tokens_bwd_kernel<<<H, pnm::kPaTokenThreads, smem, (cudaStream_t)stream>>>(pnm::make_src(srcs, world, use_flags), Wqkv, Wo,
                                                                   pnm::make_saved(saved), dWo, dWqkv, d_norm,
                                                                   (__nv_bfloat16*)Bcat16, (__nv_bfloat16*)BdT16, H, D, Cout,
                                                                   scale, share, p, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int pnm_pa_prepare_bwd(const float* dWc, const float* dbc, const float* grp, const float* Wx, const float* bx, const float* Ws,
                       const float* temp, float* dWx, float* dbx, float* dWs, float* dbs, float* dtemp, int H, int D, int C,
                       void* stream) {
  if (H <= 0 || D <= 0 || D > pnm::kPaMaxD || C <= 0) return -2;
  pnm::pa_prepare_bwd_kernel<<<H * D + (pnm::kPaS * D) / 8 + 1, 256, 0, (cudaStream_t)stream>>>(dWc, dbc, grp, Wx, bx, Ws, temp, dWx, dbx,
                                                                                      dWs, dbs, dtemp, H, D, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
