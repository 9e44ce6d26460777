// Headless renderers: every kernel writes plain RGBA / depth / normal tensors; no graphics API is involved.
//
//   volume ray-march        one thread per pixel, trilinear RGBA sampling, front-to-back compositing, early exit
//   isosurface              one thread per pixel, ray-march to the first sign change, linear refinement, gradient normal
//   mesh ray-cast           one thread per pixel, first hit through the implicit BVH, barycentric colours, Lambert shading
//   point cloud / wireframe two passes: splat a packed (depth, id) key per covered pixel with a 64-bit atomic min,
//                           then resolve the winner of every pixel
//   line integral conv.     one thread per voxel, midpoint streamline integration in both directions
//   colour maps             scalar / vector magnitude -> jet colour + opacity, 4 bytes per voxel
//
// Camera = {eye, forward, right, up} (4 x float3); pixel (x, y) looks along
// normalize(forward + px * right + py * up), px = ((x+.5)/W*2-1) * tan(fov/2) * aspect, py = (1-(y+.5)/H*2) * tan(fov/2).
#include <cuda_runtime.h>
#include <stdint.h>

#include "bvh_device.cuh"
#include "pnm_api.h"

namespace pnm {

constexpr float kFar = 3.402823e38f;

struct Camera { F3 eye, fwd, right, up; };

__device__ __forceinline__ Camera load_camera(const float* c) {
  Camera k;
  k.eye = ld3(c); k.fwd = ld3(c + 3); k.right = ld3(c + 6); k.up = ld3(c + 9);
  return k;
}

__device__ __forceinline__ F3 normalize3(F3 v) {
  const float l = sqrtf(dot(v, v));
  return l <= 1e-12f ? mk(0.f, 0.f, 0.f) : v * (1.f / l);
}

__device__ __forceinline__ F3 pixel_ray(int tid, int W, int H, const Camera& cam, float tan_half, float aspect) {
  const int y = tid / W, x = tid - y * W;
  const float px = (((float)x + 0.5f) / (float)W * 2.f - 1.f) * tan_half * aspect;
  const float py = (1.f - ((float)y + 0.5f) / (float)H * 2.f) * tan_half;
  return normalize3(cam.fwd + cam.right * px + cam.up * py);
}

// slab test against [lo, hi]; returns false on a miss, else [t_near (>= 0), t_far]
__device__ __forceinline__ bool ray_bounds(F3 o, F3 d, F3 lo, F3 hi, float& t_near, float& t_far) {
  const float oo[3] = {o.x, o.y, o.z}, dd[3] = {d.x, d.y, d.z}, l[3] = {lo.x, lo.y, lo.z}, h[3] = {hi.x, hi.y, hi.z};
  float tn = 0.f, tf = kFar;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    if (fabsf(dd[a]) < 1e-12f) {
      if (oo[a] < l[a] || oo[a] > h[a]) return false;
    } else {
      const float inv = 1.f / dd[a];
      const float t0 = (l[a] - oo[a]) * inv, t1 = (h[a] - oo[a]) * inv;
      tn = fmaxf(tn, fminf(t0, t1));
      tf = fminf(tf, fmaxf(t0, t1));
    }
  }
  t_near = tn; t_far = tf;
  return tf >= tn;
}

struct Cell { int i0, j0, k0; float fx, fy, fz; };

// cell and weights of a world-space point in an (nx, ny, nz) vertex grid spanning [lo, hi]
__device__ __forceinline__ Cell locate(F3 p, F3 lo, F3 hi, int nx, int ny, int nz) {
  const float sx = (p.x - lo.x) / (hi.x - lo.x) * (float)(nx - 1);
  const float sy = (p.y - lo.y) / (hi.y - lo.y) * (float)(ny - 1);
  const float sz = (p.z - lo.z) / (hi.z - lo.z) * (float)(nz - 1);
  Cell c;
  c.i0 = min(max((int)floorf(sx), 0), nx - 2);
  c.j0 = min(max((int)floorf(sy), 0), ny - 2);
  c.k0 = min(max((int)floorf(sz), 0), nz - 2);
  c.fx = fminf(fmaxf(sx - (float)c.i0, 0.f), 1.f);
  c.fy = fminf(fmaxf(sy - (float)c.j0, 0.f), 1.f);
  c.fz = fminf(fmaxf(sz - (float)c.k0, 0.f), 1.f);
  return c;
}

__device__ __forceinline__ float lerp3(float c000, float c100, float c010, float c110, float c001, float c101, float c011,
                                       float c111, float fx, float fy, float fz) {
  const float c00 = c000 * (1.f - fx) + c100 * fx, c10 = c010 * (1.f - fx) + c110 * fx;
  const float c01 = c001 * (1.f - fx) + c101 * fx, c11 = c011 * (1.f - fx) + c111 * fx;
  const float c0 = c00 * (1.f - fy) + c10 * fy, c1 = c01 * (1.f - fy) + c11 * fy;
  return c0 * (1.f - fz) + c1 * fz;
}

__device__ __forceinline__ float sample_scalar(const float* __restrict__ f, F3 p, F3 lo, F3 hi, int nx, int ny, int nz) {
  const Cell c = locate(p, lo, hi, nx, ny, nz);
  const long long sy = nz, sx = (long long)ny * nz;
  const float* b = f + c.i0 * sx + c.j0 * sy + c.k0;
  return lerp3(b[0], b[sx], b[sy], b[sx + sy], b[1], b[sx + 1], b[sy + 1], b[sx + sy + 1], c.fx, c.fy, c.fz);
}

// channels-last RGBA volume: the four channels of a vertex are one 16-byte load
__device__ __forceinline__ float4 sample_rgba(const float4* __restrict__ v, F3 p, F3 lo, F3 hi, int nx, int ny, int nz) {
  const Cell c = locate(p, lo, hi, nx, ny, nz);
  const long long sy = nz, sx = (long long)ny * nz;
  const float4* b = v + c.i0 * sx + c.j0 * sy + c.k0;
  const float4 a000 = __ldg(b), a100 = __ldg(b + sx), a010 = __ldg(b + sy), a110 = __ldg(b + sx + sy);
  const float4 a001 = __ldg(b + 1), a101 = __ldg(b + sx + 1), a011 = __ldg(b + sy + 1), a111 = __ldg(b + sx + sy + 1);
  float4 r;
  r.x = lerp3(a000.x, a100.x, a010.x, a110.x, a001.x, a101.x, a011.x, a111.x, c.fx, c.fy, c.fz);
  r.y = lerp3(a000.y, a100.y, a010.y, a110.y, a001.y, a101.y, a011.y, a111.y, c.fx, c.fy, c.fz);
  r.z = lerp3(a000.z, a100.z, a010.z, a110.z, a001.z, a101.z, a011.z, a111.z, c.fx, c.fy, c.fz);
  r.w = lerp3(a000.w, a100.w, a010.w, a110.w, a001.w, a101.w, a011.w, a111.w, c.fx, c.fy, c.fz);
  return r;
}

__device__ __forceinline__ float4 shade(float4 c, F3 n, F3 light, float ambient) {
  const float k = ambient + (1.f - ambient) * fmaxf(dot(n, light), 0.f);
  return make_float4(c.x * k, c.y * k, c.z * k, c.w);
}

__global__ void volume_render_kernel(const float4* __restrict__ vol, const float* __restrict__ camera,
                                     const float* __restrict__ bounds, int W, int H, float step, int max_steps, float tan_half,
                                     float aspect, float opacity_stop, float depth_thr, int nx, int ny, int nz,
                                     float4* __restrict__ rgba, float* __restrict__ depth) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= W * H) return;
  const Camera cam = load_camera(camera);
  const F3 d = pixel_ray(tid, W, H, cam, tan_half, aspect);
  const F3 lo = ld3(bounds), hi = ld3(bounds + 3);
  float tn, tf;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float first = kFar;
  if (ray_bounds(cam.eye, d, lo, hi, tn, tf)) {
    float t = tn;
    for (int s = 0; s < max_steps; ++s) {
      if (t > tf || acc.w >= opacity_stop) break;
      const float4 smp = sample_rgba(vol, cam.eye + d * t, lo, hi, nx, ny, nz);
      const float a = fminf(fmaxf(smp.w, 0.f), 1.f);
      if (a > 0.f) {
        const float o = (1.f - acc.w) * a;
        acc.x += smp.x * o; acc.y += smp.y * o; acc.z += smp.z * o; acc.w += o;
        if (first >= 3.0e38f && acc.w >= depth_thr) first = t;
      }
      t += step;
    }
  }
  if (acc.w <= 0.f) {
    rgba[tid] = make_float4(0.f, 0.f, 0.f, 0.f);
    depth[tid] = kFar;
  } else {
    const float inv = 1.f / acc.w;
    rgba[tid] = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w);
    depth[tid] = first;
  }
}

__global__ void isosurface_render_kernel(const float* __restrict__ field, const float4* __restrict__ color_field,
                                         const float* __restrict__ camera, const float* __restrict__ bounds,
                                         const float* __restrict__ uniform_color, const float* __restrict__ light, int W, int H,
                                         float threshold, float step, int max_steps, float tan_half, float aspect,
                                         float ambient, int has_color_field, int nx, int ny, int nz, float4* __restrict__ rgba,
                                         float* __restrict__ depth, float* __restrict__ normal_out) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= W * H) return;
  const Camera cam = load_camera(camera);
  const F3 d = pixel_ray(tid, W, H, cam, tan_half, aspect);
  const F3 lo = ld3(bounds), hi = ld3(bounds + 3);
  float tn, tf, hit_t = kFar;
  bool found = false;
  if (ray_bounds(cam.eye, d, lo, hi, tn, tf)) {
    float pt = tn, pv = sample_scalar(field, cam.eye + d * tn, lo, hi, nx, ny, nz);
    for (int s = 0; s < max_steps && !found; ++s) {
      const float nt = pt + step;
      if (nt > tf) break;
      const float nv = sample_scalar(field, cam.eye + d * nt, lo, hi, nx, ny, nz);
      if ((pv - threshold) * (nv - threshold) <= 0.f) {
        float den = nv - pv;
        if (fabsf(den) < 1e-7f) den = den < 0.f ? -1e-7f : 1e-7f;
        hit_t = pt + fminf(fmaxf((threshold - pv) / den, 0.f), 1.f) * step;
        found = true;
      }
      pt = nt; pv = nv;
    }
  }
  if (!found) {
    rgba[tid] = make_float4(0.f, 0.f, 0.f, 0.f);
    depth[tid] = kFar;
    normal_out[3 * tid] = normal_out[3 * tid + 1] = normal_out[3 * tid + 2] = 0.f;
    return;
  }
  const F3 p = cam.eye + d * hit_t;
  const float dx = (hi.x - lo.x) / (float)(nx - 1), dy = (hi.y - lo.y) / (float)(ny - 1), dz = (hi.z - lo.z) / (float)(nz - 1);
  F3 g;
  g.x = (sample_scalar(field, p + mk(0.5f * dx, 0, 0), lo, hi, nx, ny, nz) - sample_scalar(field, p - mk(0.5f * dx, 0, 0), lo, hi, nx, ny, nz)) / dx;
  g.y = (sample_scalar(field, p + mk(0, 0.5f * dy, 0), lo, hi, nx, ny, nz) - sample_scalar(field, p - mk(0, 0.5f * dy, 0), lo, hi, nx, ny, nz)) / dy;
  g.z = (sample_scalar(field, p + mk(0, 0, 0.5f * dz), lo, hi, nx, ny, nz) - sample_scalar(field, p - mk(0, 0, 0.5f * dz), lo, hi, nx, ny, nz)) / dz;
  F3 n = normalize3(g);
  if (dot(n, d) > 0.f) n = n * -1.f;
  float4 c = make_float4(uniform_color[0], uniform_color[1], uniform_color[2], uniform_color[3]);
  if (has_color_field) c = sample_rgba(color_field, p, lo, hi, nx, ny, nz);
  rgba[tid] = shade(c, n, ld3(light), ambient);
  depth[tid] = hit_t;
  normal_out[3 * tid] = n.x; normal_out[3 * tid + 1] = n.y; normal_out[3 * tid + 2] = n.z;
}

// color_mode: 0 uniform, 1 per-vertex (interpolated), 2 per-face
__global__ void mesh_raycast_kernel(const float* __restrict__ bvh_bounds, const int* __restrict__ order,
                                    const float* __restrict__ tris, const int* __restrict__ indices, int n_leaves,
                                    const float* __restrict__ colors, const float* __restrict__ camera,
                                    const float* __restrict__ uniform_color, const float* __restrict__ light, int W, int H,
                                    float tan_half, float aspect, float max_distance, float ambient, int color_mode,
                                    float4* __restrict__ rgba, float* __restrict__ depth, float* __restrict__ normal_out) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= W * H) return;
  const Camera cam = load_camera(camera);
  const F3 d = pixel_ray(tid, W, H, cam, tan_half, aspect);
  int face;
  float u, v;
  const float t = bvh_trace(bvh_bounds, order, tris, n_leaves, cam.eye, d, max_distance, face, u, v);
  if (face < 0) {
    rgba[tid] = make_float4(0.f, 0.f, 0.f, 0.f);
    depth[tid] = kFar;
    normal_out[3 * tid] = normal_out[3 * tid + 1] = normal_out[3 * tid + 2] = 0.f;
    return;
  }
  const float* T = tris + 9LL * face;
  const F3 v0 = ld3(T);
  F3 n = normalize3(cross(ld3(T + 3) - v0, ld3(T + 6) - v0));
  if (dot(n, d) > 0.f) n = n * -1.f;
  float4 c = make_float4(uniform_color[0], uniform_color[1], uniform_color[2], uniform_color[3]);
  if (color_mode == 1) {
    const float w0 = 1.f - u - v;
    const float* c0 = colors + 4LL * indices[3 * face];
    const float* c1 = colors + 4LL * indices[3 * face + 1];
    const float* c2 = colors + 4LL * indices[3 * face + 2];
    c = make_float4(w0 * c0[0] + u * c1[0] + v * c2[0], w0 * c0[1] + u * c1[1] + v * c2[1],
                    w0 * c0[2] + u * c1[2] + v * c2[2], w0 * c0[3] + u * c1[3] + v * c2[3]);
  } else if (color_mode == 2) {
    const float* cf = colors + 4LL * face;
    c = make_float4(cf[0], cf[1], cf[2], cf[3]);
  }
  rgba[tid] = shade(c, n, ld3(light), ambient);
  depth[tid] = t;
  normal_out[3 * tid] = n.x; normal_out[3 * tid + 1] = n.y; normal_out[3 * tid + 2] = n.z;
}

__device__ __forceinline__ void splat(long long* winners, int x, int y, int W, int H, long long key) {
  if (x >= 0 && x < W && y >= 0 && y < H) atomicMin(winners + (long long)y * W + x, key);
}

__global__ void point_depth_kernel(const float* __restrict__ points, const float* __restrict__ camera, int W, int H,
                                   float tan_half, float aspect, float z_near, float z_far, int point_size, long long n,
                                   float depth_scale, long long* __restrict__ winners) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tid >= n) return;
  const Camera cam = load_camera(camera);
  const F3 rel = ld3(points + 3 * tid) - cam.eye;
  const float z = dot(rel, cam.fwd);
  if (z <= z_near || z >= z_far || z <= 1e-12f) return;
  const float sx = (dot(rel, cam.right) / (z * tan_half * aspect) + 1.f) * 0.5f * (float)W;
  const float sy = (1.f - (dot(rel, cam.up) / (z * tan_half) + 1.f) * 0.5f) * (float)H;
  if (!(fabsf(sx) < 1e9f) || !(fabsf(sy) < 1e9f)) return;
  const int cx = (int)sx, cy = (int)sy, r = point_size / 2;
  const long long key = (long long)(z * depth_scale) * n + tid;
  for (int dy = -r; dy <= r; ++dy)
    for (int dx = -r; dx <= r; ++dx) splat(winners, cx + dx, cy + dy, W, H, key);
}

__global__ void point_resolve_kernel(const float* __restrict__ points, const float* __restrict__ colors,
                                     const float* __restrict__ camera, const float* __restrict__ uniform_color, int W, int H,
                                     int has_colors, long long n, long long empty_key, const long long* __restrict__ winners,
                                     float4* __restrict__ rgba, float* __restrict__ depth) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= W * H) return;
  const long long key = winners[tid];
  if (key == empty_key) return;
  const long long id = key % n;
  const Camera cam = load_camera(camera);
  const float* c = has_colors ? colors + 4 * id : uniform_color;
  rgba[tid] = make_float4(c[0], c[1], c[2], c[3]);
  depth[tid] = dot(ld3(points + 3 * id) - cam.eye, cam.fwd);
}

__global__ void wire_depth_kernel(const float* __restrict__ edges, const float* __restrict__ camera, int W, int H,
                                  float tan_half, float aspect, float z_near, float z_far, int thickness, long long n,
                                  float depth_scale, long long* __restrict__ winners) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tid >= n) return;
  const Camera cam = load_camera(camera);
  F3 p0 = ld3(edges + 6 * tid), p1 = ld3(edges + 6 * tid + 3);
  float z0 = dot(p0 - cam.eye, cam.fwd), z1 = dot(p1 - cam.eye, cam.fwd);
  if ((z0 <= z_near && z1 <= z_near) || (z0 >= z_far && z1 >= z_far)) return;
  if (z0 < z_near) { p0 = p0 + (p1 - p0) * ((z_near - z0) / (z1 - z0)); z0 = z_near; }
  else if (z1 < z_near) { p1 = p1 + (p0 - p1) * ((z_near - z1) / (z0 - z1)); z1 = z_near; }
  if (z0 > z_far) { p0 = p0 + (p1 - p0) * ((z_far - z0) / (z1 - z0)); z0 = z_far; }
  else if (z1 > z_far) { p1 = p1 + (p0 - p1) * ((z_far - z1) / (z0 - z1)); z1 = z_far; }
  const F3 r0 = p0 - cam.eye, r1 = p1 - cam.eye;
  const float fx0 = (dot(r0, cam.right) / (z0 * tan_half * aspect) + 1.f) * 0.5f * (float)W;
  const float fy0 = (1.f - (dot(r0, cam.up) / (z0 * tan_half) + 1.f) * 0.5f) * (float)H;
  const float fx1 = (dot(r1, cam.right) / (z1 * tan_half * aspect) + 1.f) * 0.5f * (float)W;
  const float fy1 = (1.f - (dot(r1, cam.up) / (z1 * tan_half) + 1.f) * 0.5f) * (float)H;
  // an endpoint far outside the image would make the walk below very long: clamp it to a margin around the image;
  // the clamped part of the segment is invisible anyway
  const float m = 4.f * (float)(W + H);
  if (!(fabsf(fx0) < 1e9f) || !(fabsf(fy0) < 1e9f) || !(fabsf(fx1) < 1e9f) || !(fabsf(fy1) < 1e9f)) return;
  int x0 = (int)fminf(fmaxf(fx0, -m), m), y0 = (int)fminf(fmaxf(fy0, -m), m);
  const int x1 = (int)fminf(fmaxf(fx1, -m), m), y1 = (int)fminf(fmaxf(fy1, -m), m);
  const int dx = abs(x1 - x0), dy = abs(y1 - y0), sx = x0 > x1 ? -1 : 1, sy = y0 > y1 ? -1 : 1;
  const int steps = max(dx, dy), r = thickness / 2;
  int err = dx - dy;
  for (int s = 0; s <= steps; ++s) {                      // Bresenham walk, depth interpolated along the major axis
    const float a = steps > 0 ? (float)s / (float)steps : 0.f;
    const float z = z0 * (1.f - a) + z1 * a;
    const long long key = (long long)(z * depth_scale) * n + tid;
    for (int oy = -r; oy <= r; ++oy)
      for (int ox = -r; ox <= r; ++ox) splat(winners, x0 + ox, y0 + oy, W, H, key);
    if (x0 == x1 && y0 == y1) break;
    const int e2 = 2 * err;
    if (e2 > -dy) { err -= dy; x0 += sx; }
    if (e2 < dx) { err += dx; y0 += sy; }
  }
}

__global__ void wire_resolve_kernel(const float* __restrict__ uniform_color, long long n, long long empty_key, float depth_scale,
                                    const long long* __restrict__ winners, int n_pix, float4* __restrict__ rgba,
                                    float* __restrict__ depth) {
  const int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (tid >= n_pix) return;
  const long long key = winners[tid];
  if (key == empty_key) return;
  rgba[tid] = make_float4(uniform_color[0], uniform_color[1], uniform_color[2], uniform_color[3]);
  depth[tid] = (float)(key / n) / depth_scale;
}

// index-space trilinear sampling with clamped neighbours (used by the streamline integrator)
__device__ __forceinline__ void index_cell(F3 p, int nx, int ny, int nz, int* i, float* f) {
  i[0] = min(max((int)floorf(p.x), 0), nx - 1); i[1] = min(max((int)floorf(p.y), 0), ny - 1);
  i[2] = min(max((int)floorf(p.z), 0), nz - 1);
  i[3] = min(i[0] + 1, nx - 1); i[4] = min(i[1] + 1, ny - 1); i[5] = min(i[2] + 1, nz - 1);
  f[0] = fminf(fmaxf(p.x - (float)i[0], 0.f), 1.f); f[1] = fminf(fmaxf(p.y - (float)i[1], 0.f), 1.f);
  f[2] = fminf(fmaxf(p.z - (float)i[2], 0.f), 1.f);
}

__device__ __forceinline__ float sample_seed(const float* __restrict__ s, F3 p, int nx, int ny, int nz) {
  int i[6]; float f[3];
  index_cell(p, nx, ny, nz, i, f);
  const long long sy = nz, sx = (long long)ny * nz;
#define AT(a, b, c) __ldg(s + i[a] * sx + i[b] * sy + i[c])
  return lerp3(AT(0, 1, 2), AT(3, 1, 2), AT(0, 4, 2), AT(3, 4, 2), AT(0, 1, 5), AT(3, 1, 5), AT(0, 4, 5), AT(3, 4, 5), f[0], f[1], f[2]);
#undef AT
}

__device__ __forceinline__ F3 sample_vec(const float* __restrict__ v, F3 p, int nx, int ny, int nz) {
  int i[6]; float f[3];
  index_cell(p, nx, ny, nz, i, f);
  const long long sy = 3LL * nz, sx = 3LL * ny * nz;
  float r[3];
#pragma unroll
  for (int ch = 0; ch < 3; ++ch) {
#define AT(a, b, c) __ldg(v + i[a] * sx + i[b] * sy + 3 * i[c] + ch)
    r[ch] = lerp3(AT(0, 1, 2), AT(3, 1, 2), AT(0, 4, 2), AT(3, 4, 2), AT(0, 1, 5), AT(3, 1, 5), AT(0, 4, 5), AT(3, 4, 5), f[0], f[1], f[2]);
#undef AT
  }
  return mk(r[0], r[1], r[2]);
}

__global__ void lic_kernel(const float* __restrict__ vec, const float* __restrict__ seed, float step, int num_steps,
                           float contrast, int nx, int ny, int nz, float* __restrict__ out) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tid >= (long long)nx * ny * nz) return;
  const int k = (int)(tid % nz), j = (int)((tid / nz) % ny), i = (int)(tid / ((long long)nz * ny));
  const F3 pos = mk((float)i, (float)j, (float)k);
  float total = seed[tid], wsum = 1.f;
  for (int dir = 0; dir < 2; ++dir) {
    const float sgn = dir ? -1.f : 1.f;
    F3 cur = pos;
    for (int s = 0; s < num_steps; ++s) {
      F3 v = sample_vec(vec, cur, nx, ny, nz);
      float l = sqrtf(dot(v, v));
      if (l <= 1e-6f) break;
      v = v * (sgn / l);
      F3 mv = sample_vec(vec, cur + v * (0.5f * step), nx, ny, nz);
      l = sqrtf(dot(mv, mv));
      if (l <= 1e-6f) break;
      cur = cur + mv * (sgn / l * step);
      if (cur.x < 0.f || cur.x > (float)(nx - 1) || cur.y < 0.f || cur.y > (float)(ny - 1) || cur.z < 0.f || cur.z > (float)(nz - 1)) break;
      const float w = 1.f - (float)(s + 1) / (float)(num_steps + 1);
      total += sample_seed(seed, cur, nx, ny, nz) * w;
      wsum += w;
    }
  }
  float val = fminf(fmaxf(total / fmaxf(wsum, 1e-6f), 0.f), 1.f);
  val = (val - 0.5f) * contrast + 0.5f;
  out[tid] = fminf(fmaxf(val, 0.f), 1.f);
}

__device__ __forceinline__ uchar4 jet_rgba(float v, float alpha) {
  const float r = fminf(fmaxf(fminf(4.f * v - 1.5f, -4.f * v + 4.5f), 0.f), 1.f);
  const float g = fminf(fmaxf(fminf(4.f * v - 0.5f, -4.f * v + 3.5f), 0.f), 1.f);
  const float b = fminf(fmaxf(fminf(4.f * v + 0.5f, -4.f * v + 2.5f), 0.f), 1.f);
  return make_uchar4((unsigned char)(r * 255.f), (unsigned char)(g * 255.f), (unsigned char)(b * 255.f),
                     (unsigned char)(fminf(fmaxf(alpha, 0.f), 1.f) * 255.f));
}

__global__ void scalar_rgba_kernel(const float* __restrict__ field, long long n, float vmin, float inv_range, float max_opacity,
                                   float opacity_threshold, uchar4* __restrict__ out) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tid >= n) return;
  const float v = fminf(fmaxf((field[tid] - vmin) * inv_range, 0.f), 1.f);
  out[tid] = jet_rgba(v, (v < opacity_threshold ? 0.f : v) * max_opacity);
}

__global__ void vector_rgba_kernel(const float* __restrict__ vec, const float* __restrict__ lic, long long n, float vmin,
                                   float inv_range, float max_opacity, float lic_threshold, uchar4* __restrict__ out) {
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (tid >= n) return;
  const F3 w = ld3(vec + 3 * tid);
  const float v = fminf(fmaxf((sqrtf(dot(w, w)) - vmin) * inv_range, 0.f), 1.f);
  float l = fminf(fmaxf(lic[tid], 0.f), 1.f);
  if (l < lic_threshold) l = 0.f;
  out[tid] = jet_rgba(v, l * v * max_opacity);
}

}  // namespace pnm

#define PNM_GRID(n) (unsigned)(((n) + 127) / 128), 128, 0, (cudaStream_t)stream

extern "C" {

int pnm_volume_render(const float* vol, const float* camera, const float* bounds, int W, int H, float step, int max_steps,
                      float tan_half, float aspect, float opacity_stop, float depth_thr, int nx, int ny, int nz, float* rgba,
                      float* depth, void* stream) {
  pnm::volume_render_kernel<<<PNM_GRID((long long)W * H)>>>((const float4*)vol, camera, bounds, W, H, step, max_steps, tan_half,
                                                             aspect, opacity_stop, depth_thr, nx, ny, nz, (float4*)rgba, depth);
  return (int)cudaGetLastError();
}

int pnm_isosurface_render(const float* field, const float* color_field, const float* camera, const float* bounds,
                          const float* uniform_color, const float* light, int W, int H, float threshold, float step,
                          int max_steps, float tan_half, float aspect, float ambient, int has_color_field, int nx, int ny,
                          int nz, float* rgba, float* depth, float* normal, void* stream) {
  pnm::isosurface_render_kernel<<<PNM_GRID((long long)W * H)>>>(field, (const float4*)color_field, camera, bounds, uniform_color,
                                                                 light, W, H, threshold, step, max_steps, tan_half, aspect,
                                                                 ambient, has_color_field, nx, ny, nz, (float4*)rgba, depth, normal);
  return (int)cudaGetLastError();
}

int pnm_mesh_raycast_render(const float* bvh_bounds, const int* order, const float* tris, const int* indices, int n_leaves,
                            const float* colors, const float* camera, const float* uniform_color, const float* light, int W,
                            int H, float tan_half, float aspect, float max_distance, float ambient, int color_mode,
                            float* rgba, float* depth, float* normal, void* stream) {
  pnm::mesh_raycast_kernel<<<PNM_GRID((long long)W * H)>>>(bvh_bounds, order, tris, indices, n_leaves, colors, camera, uniform_color,
                                                            light, W, H, tan_half, aspect, max_distance, ambient, color_mode,
                                                            (float4*)rgba, depth, normal);
  return (int)cudaGetLastError();
}

int pnm_point_cloud_render(const float* points, const float* colors, const float* camera, const float* uniform_color, int W,
                           int H, float tan_half, float aspect, float z_near, float z_far, int point_size, long long n,
                           float depth_scale, long long empty_key, int has_colors, long long* winners, float* rgba,
                           float* depth, void* stream) {
  pnm::point_depth_kernel<<<PNM_GRID(n)>>>(points, camera, W, H, tan_half, aspect, z_near, z_far, point_size, n, depth_scale, winners);
  pnm::point_resolve_kernel<<<PNM_GRID((long long)W * H)>>>(points, colors, camera, uniform_color, W, H, has_colors, n, empty_key,
                                                             winners, (float4*)rgba, depth);
  return (int)cudaGetLastError();
}

int pnm_wireframe_render(const float* edges, const float* camera, const float* uniform_color, int W, int H, float tan_half,
                         float aspect, float z_near, float z_far, int thickness, long long n, float depth_scale,
                         long long empty_key, long long* winners, float* rgba, float* depth, void* stream) {
  pnm::wire_depth_kernel<<<PNM_GRID(n)>>>(edges, camera, W, H, tan_half, aspect, z_near, z_far, thickness, n, depth_scale, winners);
  pnm::wire_resolve_kernel<<<PNM_GRID((long long)W * H)>>>(uniform_color, n, empty_key, depth_scale, winners, W * H, (float4*)rgba, depth);
  return (int)cudaGetLastError();
}

int pnm_line_integral_convolution(const float* vec, const float* seed, float step, int num_steps, float contrast, int nx,
                                  int ny, int nz, float* out, void* stream) {
  pnm::lic_kernel<<<PNM_GRID((long long)nx * ny * nz)>>>(vec, seed, step, num_steps, contrast, nx, ny, nz, out);
  return (int)cudaGetLastError();
}

int pnm_scalar_field_to_rgba(const float* field, long long n, float vmin, float vmax, float max_opacity,
                             float opacity_threshold, unsigned char* out, void* stream) {
  if (n <= 0) return 0;
  pnm::scalar_rgba_kernel<<<PNM_GRID(n)>>>(field, n, vmin, 1.f / (vmax - vmin), max_opacity, opacity_threshold, (uchar4*)out);
  return (int)cudaGetLastError();
}

int pnm_vector_field_to_rgba(const float* vec, const float* lic, long long n, float vmin, float vmax, float max_opacity,
                             float lic_threshold, unsigned char* out, void* stream) {
  if (n <= 0) return 0;
  pnm::vector_rgba_kernel<<<PNM_GRID(n)>>>(vec, lic, n, vmin, 1.f / (vmax - vmin), max_opacity, lic_threshold, (uchar4*)out);
  return (int)cudaGetLastError();
}

}  // extern "C"
