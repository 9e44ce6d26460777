// Periodic finite-difference "stencil programs" on 1-3-D grids.
//
// One kernel evaluates any linear periodic stencil operator
//     out[oc][p] = sum_t coef_t(p) * in[ic_t][(p + shift_t) mod n]
// where a term's coefficient is a constant or a per-index table along one axis (non-uniform
// spacing).  Gradients, divergence, curl, Laplacians, mixed second derivatives, orders 2 and 4,
// and every backward pass (the transposed program) are instances; the host builds the term list.
// One thread per grid point, all output channels per thread, so the input is read from DRAM
// once and the neighbours come from L1/L2.
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"

namespace pnm {

constexpr int kMaxTerms = 112;

struct StencilTerm {
  float coef;       // constant factor (multiplies the table value when tab >= 0)
  int8_t oc, ic;    // output / input channel
  int8_t s0, s1, s2;  // shift along each grid axis
  int8_t tab;       // -1: none, else index of the coefficient table (see tab_axis)
  int8_t tab_axis;  // grid axis the table is indexed by
  int8_t at_src;    // 1: index the table at the shifted (source) position, 0: at the output position
};
static_assert(sizeof(StencilTerm) == 12, "layout shared with the Python side");

struct StencilProgram {
  StencilTerm terms[kMaxTerms];
  int n_terms, n_out, n_in, ndim;
  int dims[3];         // grid extents (unused axes = 1)
  long long tab_off[12];  // start of each table inside `tables`
};

__device__ __forceinline__ int wrap(int i, int n) {
  i %= n;
  return i < 0 ? i + n : i;
}

template <typename T>
__global__ void __launch_bounds__(256)
stencil_program_kernel(const T* __restrict__ in, T* __restrict__ out, const T* __restrict__ tables,
                       const __grid_constant__ StencilProgram prog, long long npts) {
  const long long p = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (p >= npts) return;
  const int n0 = prog.dims[0], n1 = prog.dims[1], n2 = prog.dims[2];
  const int i2 = int(p % n2);
  const int i1 = int((p / n2) % n1);
  const int i0 = int(p / ((long long)n2 * n1));
  // terms are sorted by output channel (checked on the host): one running sum, stored when the channel changes
  T acc = T(0);
  int cur = 0;
  for (int t = 0; t < prog.n_terms; ++t) {
    const StencilTerm tm = prog.terms[t];
    while (cur < tm.oc) {
      out[(long long)cur * npts + p] = acc;
      acc = T(0);
      ++cur;
    }
    const int j0 = tm.s0 ? wrap(i0 + tm.s0, n0) : i0;
    const int j1 = tm.s1 ? wrap(i1 + tm.s1, n1) : i1;
    const int j2 = tm.s2 ? wrap(i2 + tm.s2, n2) : i2;
    T c = T(tm.coef);
    if (tm.tab >= 0) {
      int idx;
      if (tm.at_src) idx = tm.tab_axis == 0 ? j0 : (tm.tab_axis == 1 ? j1 : j2);
      else idx = tm.tab_axis == 0 ? i0 : (tm.tab_axis == 1 ? i1 : i2);
      c *= tables[prog.tab_off[tm.tab] + idx];
    }
    acc += c * in[(long long)tm.ic * npts + ((long long)j0 * n1 + j1) * n2 + j2];
  }
  for (; cur < prog.n_out; ++cur) {
    out[(long long)cur * npts + p] = acc;
    acc = T(0);
  }
}

}  // namespace pnm

extern "C" {

int pnm_stencil_max_terms() { return pnm::kMaxTerms; }
int pnm_stencil_program_bytes() { return (int)sizeof(pnm::StencilProgram); }

// prog: host pointer to a StencilProgram; in: [n_in, npts], out: [n_out, npts]; dtype 0 = fp32, 1 = fp64.
int pnm_stencil_apply(const void* in, void* out, const void* tables, const void* prog_host, int dtype, void* stream) {
  const pnm::StencilProgram& prog = *reinterpret_cast<const pnm::StencilProgram*>(prog_host);
  if (prog.n_terms > pnm::kMaxTerms || prog.n_out < 1) return -1;
  for (int t = 1; t < prog.n_terms; ++t)
    if (prog.terms[t].oc < prog.terms[t - 1].oc) return -3;
  const long long npts = (long long)prog.dims[0] * prog.dims[1] * prog.dims[2];
  if (npts <= 0) return 0;
  const int threads = 256;
  const long long blocks = (npts + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return -2;
  if (dtype == 0)
    pnm::stencil_program_kernel<float><<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
        (const float*)in, (float*)out, (const float*)tables, prog, npts);
  else
    pnm::stencil_program_kernel<double><<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
        (const double*)in, (double*)out, (const double*)tables, prog, npts);
  return (int)cudaGetLastError();
}

}  // extern "C"
