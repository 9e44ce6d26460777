// Device-side pieces shared by the mesh query kernels and the renderers: a small float3, the ray / box slab test,
// and first-hit traversal of the implicit BVH (node i -> children 2i+1, 2i+2; leaves start at node L-1).
#pragma once
#include <cuda_runtime.h>

namespace pnm {

constexpr int kStack = 64;

struct F3 { float x, y, z; };
__device__ __forceinline__ F3 mk(float x, float y, float z) { F3 r; r.x = x; r.y = y; r.z = z; return r; }
__device__ __forceinline__ F3 operator-(F3 a, F3 b) { return mk(a.x - b.x, a.y - b.y, a.z - b.z); }
__device__ __forceinline__ F3 operator+(F3 a, F3 b) { return mk(a.x + b.x, a.y + b.y, a.z + b.z); }
__device__ __forceinline__ F3 operator*(F3 a, float s) { return mk(a.x * s, a.y * s, a.z * s); }
__device__ __forceinline__ float dot(F3 a, F3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ F3 cross(F3 a, F3 b) { return mk(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }
__device__ __forceinline__ F3 ld3(const float* p) { return mk(p[0], p[1], p[2]); }

__device__ __forceinline__ bool ray_box(const float* b, F3 o, F3 inv, float tmax, float& tnear) {
  float t0 = 0.f, t1 = tmax;
  const float lo[3] = {b[0], b[1], b[2]}, hi[3] = {b[3], b[4], b[5]};
  const float oo[3] = {o.x, o.y, o.z}, ii[3] = {inv.x, inv.y, inv.z};
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    float ta = (lo[a] - oo[a]) * ii[a], tb = (hi[a] - oo[a]) * ii[a];
    if (ta > tb) { const float s = ta; ta = tb; tb = s; }
    t0 = fmaxf(t0, ta);
    t1 = fminf(t1, tb);
  }
  tnear = t0;
  return t0 <= t1;
}

// First hit of the ray o + t d (d normalised) with t in (1e-9, max_distance).  Returns t (max_distance on a miss);
// face = -1 on a miss; (u, v) are the barycentric weights of the triangle's second and third vertex.
__device__ __forceinline__ float bvh_trace(const float* __restrict__ bounds, const int* __restrict__ order,
                                           const float* __restrict__ tris, int n_leaves, F3 o, F3 d, float max_distance,
                                           int& face, float& bu, float& bv) {
  const float big = 1e30f;
  const F3 inv = mk(fabsf(d.x) > 1e-20f ? 1.f / d.x : copysignf(big, d.x), fabsf(d.y) > 1e-20f ? 1.f / d.y : copysignf(big, d.y),
                    fabsf(d.z) > 1e-20f ? 1.f / d.z : copysignf(big, d.z));
  float best = max_distance;
  bu = bv = 0.f;
  int best_face = -1;
  int stack[kStack];
  int sp = 0;
  stack[sp++] = 0;
  const int first_leaf = n_leaves - 1;
  while (sp > 0) {
    const int node = stack[--sp];
    float tn;
    if (!ray_box(bounds + 6 * node, o, inv, best, tn)) continue;
    if (node >= first_leaf) {
      const int t = order[node - first_leaf];
      if (t < 0) continue;
      const float* T = tris + 9LL * t;
      const F3 v0 = ld3(T), e1 = ld3(T + 3) - v0, e2 = ld3(T + 6) - v0;
      const F3 pv = cross(d, e2);
      const float det = dot(e1, pv);
      if (fabsf(det) < 1e-12f) continue;
      const float idet = 1.f / det;
      const F3 tv = o - v0;
      const float u = dot(tv, pv) * idet;
      if (u < 0.f || u > 1.f) continue;
      const F3 qv = cross(tv, e1);
      const float v = dot(d, qv) * idet;
      if (v < 0.f || u + v > 1.f) continue;
      const float tt = dot(e2, qv) * idet;
      if (tt > 1e-9f && tt < best) { best = tt; best_face = t; bu = u; bv = v; }
      continue;
    }
    const int l = 2 * node + 1, r = l + 1;
    float tl, tr;
    const bool hl = ray_box(bounds + 6 * l, o, inv, best, tl), hr = ray_box(bounds + 6 * r, o, inv, best, tr);
    if (hl && hr) {
      if (tl < tr) { if (sp < kStack) stack[sp++] = r; if (sp < kStack) stack[sp++] = l; }
      else { if (sp < kStack) stack[sp++] = l; if (sp < kStack) stack[sp++] = r; }
    } else if (hl) { if (sp < kStack) stack[sp++] = l; }
    else if (hr) { if (sp < kStack) stack[sp++] = r; }
  }
  face = best_face;
  return best;
}

}  // namespace pnm
