// Triangle-mesh queries over an implicit (complete binary, Morton-ordered) bounding-volume hierarchy:
// closest point / distance, first ray hit, and the generalised winding number.
//
// Tree layout (built on the host side with tensor ops): node i has children 2i+1 and 2i+2; the L leaves
// (L a power of two) start at node L-1; bounds[node] = {min xyz, max xyz}; order[leaf] = triangle index or -1.
// One thread per query, explicit stack (depth <= 2*log2 L), nearest-child-first descent with pruning.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "bvh_device.cuh"
#include "pnm_api.h"

namespace pnm {


__device__ __forceinline__ float box_dist2(const float* b, F3 p) {
  const float dx = fmaxf(fmaxf(b[0] - p.x, 0.f), p.x - b[3]);
  const float dy = fmaxf(fmaxf(b[1] - p.y, 0.f), p.y - b[4]);
  const float dz = fmaxf(fmaxf(b[2] - p.z, 0.f), p.z - b[5]);
  return dx * dx + dy * dy + dz * dz;
}

// closest point of triangle (a, b, c) to p (region classification)
__device__ __forceinline__ F3 closest_on_triangle(F3 p, F3 a, F3 b, F3 c) {
  const F3 ab = b - a, ac = c - a, ap = p - a;
  const float d1 = dot(ab, ap), d2 = dot(ac, ap);
  if (d1 <= 0.f && d2 <= 0.f) return a;
  const F3 bp = p - b;
  const float d3 = dot(ab, bp), d4 = dot(ac, bp);
  if (d3 >= 0.f && d4 <= d3) return b;
  const float vc = d1 * d4 - d3 * d2;
  if (vc <= 0.f && d1 >= 0.f && d3 <= 0.f) return a + ab * (d1 / (d1 - d3));
  const F3 cp = p - c;
  const float d5 = dot(ab, cp), d6 = dot(ac, cp);
  if (d6 >= 0.f && d5 <= d6) return c;
  const float vb = d5 * d2 - d1 * d6;
  if (vb <= 0.f && d2 >= 0.f && d6 <= 0.f) return a + ac * (d2 / (d2 - d6));
  const float va = d3 * d6 - d5 * d4;
  if (va <= 0.f && (d4 - d3) >= 0.f && (d5 - d6) >= 0.f) return b + (c - b) * ((d4 - d3) / ((d4 - d3) + (d5 - d6)));
  const float denom = 1.f / (va + vb + vc);
  return a + ab * (vb * denom) + ac * (vc * denom);
}


__global__ void bvh_closest_kernel(const float* __restrict__ bounds, const int* __restrict__ order,
                                   const float* __restrict__ tris, const float* __restrict__ queries,
                                   float* __restrict__ out_dist, float* __restrict__ out_point, long long* __restrict__ out_face,
                                   int n_leaves, long long nq, float max_dist) {
  const long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (q >= nq) return;
  const F3 p = ld3(queries + 3 * q);
  float best = max_dist * max_dist;
  F3 best_pt = mk(0.f, 0.f, 0.f);
  int best_face = -1;
  int stack[kStack];
  int sp = 0;
  stack[sp++] = 0;
  const int first_leaf = n_leaves - 1;
  while (sp > 0) {
    const int node = stack[--sp];
    if (box_dist2(bounds + 6 * node, p) >= best) continue;
    if (node >= first_leaf) {
      const int t = order[node - first_leaf];
      if (t < 0) continue;
      const float* T = tris + 9LL * t;
      const F3 cp = closest_on_triangle(p, ld3(T), ld3(T + 3), ld3(T + 6));
      const F3 d = p - cp;
      const float d2 = dot(d, d);
      if (d2 < best) { best = d2; best_pt = cp; best_face = t; }
      continue;
    }
    const int l = 2 * node + 1, r = l + 1;
    const float dl = box_dist2(bounds + 6 * l, p), dr = box_dist2(bounds + 6 * r, p);
    // push the farther child first so the nearer one is visited next
    if (dl < dr) {
      if (dr < best && sp < kStack) stack[sp++] = r;
      if (dl < best && sp < kStack) stack[sp++] = l;
    } else {
      if (dl < best && sp < kStack) stack[sp++] = l;
      if (dr < best && sp < kStack) stack[sp++] = r;
    }
  }
  const float nanv = __int_as_float(0x7fc00000);
  out_face[q] = best_face;
  out_dist[q] = best_face >= 0 ? sqrtf(best) : nanv;
  out_point[3 * q] = best_face >= 0 ? best_pt.x : nanv;
  out_point[3 * q + 1] = best_face >= 0 ? best_pt.y : nanv;
  out_point[3 * q + 2] = best_face >= 0 ? best_pt.z : nanv;
}


// out_t: hit distance (inf on miss); out_face: -1 on miss; out_uv: barycentric (u, v) of the hit
__global__ void bvh_raycast_kernel(const float* __restrict__ bounds, const int* __restrict__ order,
                                   const float* __restrict__ tris, const float* __restrict__ origins,
                                   const float* __restrict__ dirs, float* __restrict__ out_t, long long* __restrict__ out_face,
                                   float* __restrict__ out_uv, int n_leaves, long long nr, float max_distance) {
  const long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (q >= nr) return;
  const F3 o = ld3(origins + 3 * q);
  F3 d = ld3(dirs + 3 * q);
  const float len = sqrtf(dot(d, d));
  d = d * (len > 0.f ? 1.f / len : 0.f);
  int best_face;
  float bu, bv;
  const float best = bvh_trace(bounds, order, tris, n_leaves, o, d, max_distance, best_face, bu, bv);
  out_face[q] = best_face;
  out_t[q] = best_face >= 0 ? best : __int_as_float(0x7f800000);
  out_uv[2 * q] = bu;
  out_uv[2 * q + 1] = bv;
}

// winding number by direct summation of signed solid angles, triangles staged through shared memory
__global__ void __launch_bounds__(128)
winding_number_kernel(const float* __restrict__ tris, const float* __restrict__ queries, float* __restrict__ out,
                      long long n_tris, long long nq) {
  __shared__ float tile[128 * 9];
  const long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const F3 p = q < nq ? ld3(queries + 3 * q) : mk(0.f, 0.f, 0.f);
  float acc = 0.f;
  for (long long base = 0; base < n_tris; base += 128) {
    const int cnt = (int)min((long long)128, n_tris - base);
    __syncthreads();
    for (int t = threadIdx.x; t < cnt * 9; t += blockDim.x) tile[t] = tris[base * 9 + t];
    __syncthreads();
    if (q < nq) {
      for (int t = 0; t < cnt; ++t) {
        const F3 a = ld3(tile + 9 * t) - p, b = ld3(tile + 9 * t + 3) - p, c = ld3(tile + 9 * t + 6) - p;
        const float la = sqrtf(dot(a, a)), lb = sqrtf(dot(b, b)), lc = sqrtf(dot(c, c));
        const float num = dot(a, cross(b, c));
        const float den = la * lb * lc + dot(a, b) * lc + dot(b, c) * la + dot(c, a) * lb;
        acc += 2.f * atan2f(num, den);
      }
    }
  }
  if (q < nq) out[q] = acc / (4.f * 3.14159265358979f);
}

}  // namespace pnm

extern "C" {

int pnm_bvh_closest(const float* bounds, const int* order, const float* tris, const float* queries, float* out_dist,
                    float* out_point, long long* out_face, int n_leaves, long long nq, float max_dist, void* stream) {
  if (nq <= 0) return 0;
  pnm::bvh_closest_kernel<<<(unsigned)((nq + 127) / 128), 128, 0, (cudaStream_t)stream>>>(bounds, order, tris, queries, out_dist,
                                                                                     out_point, out_face, n_leaves, nq, max_dist);
  return (int)cudaGetLastError();
}

int pnm_bvh_raycast(const float* bounds, const int* order, const float* tris, const float* origins, const float* dirs,
                    float* out_t, long long* out_face, float* out_uv, int n_leaves, long long nr, float max_distance,
                    void* stream) {
  if (nr <= 0) return 0;
  pnm::bvh_raycast_kernel<<<(unsigned)((nr + 127) / 128), 128, 0, (cudaStream_t)stream>>>(bounds, order, tris, origins, dirs, out_t,
                                                                                     out_face, out_uv, n_leaves, nr, max_distance);
  return (int)cudaGetLastError();
}

int pnm_winding_number(const float* tris, const float* queries, float* out, long long n_tris, long long nq, void* stream) {
  if (nq <= 0) return 0;
  pnm::winding_number_kernel<<<(unsigned)((nq + 127) / 128), 128, 0, (cudaStream_t)stream>>>(tris, queries, out, n_tris, nq);
  return (int)cudaGetLastError();
}

}  // extern "C"
