// Single translation unit of the sm_100a kernel library.  Exposes a plain C ABI (raw device
// pointers + a CUDA stream) that the Python layer binds with ctypes; no dependency on the
// PyTorch headers, so the whole library rebuilds in seconds.
#include <algorithm>
#include <cstdlib>
#include "common.cuh"
#include "tmap.cuh"
#include "gemm_tn.cuh"
#include "gemm_tn_pair.cuh"
#include "gemm_nt.cuh"
#include "gemm_nt_pair.cuh"
#include "norm.cuh"
#include "graph.cuh"
#include "peer.cuh"
#include "flash_attn.cuh"
#include "pnm_api.h"

#include "pnm_internal.h"

__device__ int pnm_error_word = 0;

namespace {
// Per-device state: a process may drive more than one GPU, and both the SM count and the address of the error word
// belong to the device that is current when a function is called.
struct DevState { int num_sms = 0; int* err_ptr = nullptr; };
DevState g_dev[pnm::kMaxDevices];
thread_local int g_num_sms = 0;
thread_local int* g_err_ptr = nullptr;

int ensure_init() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= pnm::kMaxDevices) return -1;
  DevState& d = g_dev[dev];
  if (d.num_sms <= 0 || !d.err_ptr) {
    if (cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&d.err_ptr), pnm_error_word) != cudaSuccess) return -1;
  }
  g_num_sms = d.num_sms;
  g_err_ptr = d.err_ptr;
  return 0;
}
}  // namespace

namespace pnm {
int current_device() {
  int dev = 0;
  return cudaGetDevice(&dev) == cudaSuccess ? dev : 0;
}
int* error_word_ptr() { return ensure_init() ? nullptr : g_err_ptr; }
int num_sms() { return ensure_init() ? 0 : g_num_sms; }
PeerArgs make_peer_args(const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats,
                        double budget_s, const void* epoch_base) {
  PeerArgs p;
  for (int r = 0; r < kPeerMaxRanks; ++r)
    p.base[r] = r < world ? reinterpret_cast<uint8_t*>(const_cast<void*>(bases[r])) : nullptr;
  p.rank = rank; p.world = world; p.epoch = epoch; p.capacity = capacity_floats;
  p.epoch_base = reinterpret_cast<const uint32_t*>(epoch_base);
  p.budget_ns = (unsigned long long)(budget_s * 1e9);
  return p;
}
}  // namespace pnm

// PNM_GEMM_PAIR=0 in the environment keeps every GEMM on the single-CTA kernel (for A/B timing).
static bool pair_gemm_enabled() {
  static int state = -1;
  if (state < 0) {
    const char* e = getenv("PNM_GEMM_PAIR");
    state = (e && e[0] == '0') ? 0 : 1;
  }
  return state == 1;
}

extern "C" {

int pnm_version() { return 100; }

int pnm_num_sms() { return ensure_init() ? -1 : g_num_sms; }

int pnm_get_error() {
  if (ensure_init()) return -1;
  int v = 0;
  if (cudaMemcpy(&v, g_err_ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return v;
}

int pnm_reset_error() {
  if (ensure_init()) return -1;
  return cudaMemset(g_err_ptr, 0, sizeof(int)) == cudaSuccess ? 0 : -1;
}

int pnm_gemm_tn(const void* A, int lda, const void* A2, int lda2, const void* A3, int lda3, const void* B, int ldb, void* C, int ldc, void* Z,
                int ldz, const void* AUX, int ldaux, int M, int N, int K, int K1, int K2, const float* bias,
                const float* scale, float* group_out, int act, int aux_mode, int scale_post, int bn, int max_ctas,
                void* stream) {
  if (ensure_init()) return -1;
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldb % 8) || (ldc % 8)) return -3;
  if (K1 <= 0 || K1 > K) K1 = K;
  if (K2 < K1 || K2 > K) K2 = K;
  if (K1 < K && ((K1 % 64) || !A2 || (lda2 % 8))) return -4;
  if (K2 < K && ((K2 % 64) || !A3 || (lda3 % 8))) return -4;
  if (Z && AUX) return -5;
  if ((aux_mode != 0) != (AUX != nullptr)) return -6;
  if (act == pnm::ACT_SOFTMAX64 && (N % 64)) return -7;
  pnm::GemmCall c;
  c.A = A; c.lda = lda; c.A2 = A2; c.lda2 = lda2; c.A3 = A3; c.lda3 = lda3; c.B = B; c.ldb = ldb; c.C = C; c.ldc = ldc;
  c.Z = Z; c.ldz = ldz; c.AUX = AUX; c.ldaux = ldaux;
  c.M = M; c.N = N; c.K = K; c.K1 = K1; c.K2 = K2;
  c.bias = bias; c.scale = scale; c.group_out = group_out;
  c.act = act; c.aux_mode = aux_mode; c.scale_post = scale_post; c.max_ctas = max_ctas;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0 && pair_gemm_enabled() && pnm::pair_gemm_applicable(c)) {
    // compute-bound shapes: 256 x 256 tiles on CTA pairs (tcgen05.mma.cta_group::2)
    if (AUX) return pnm::launch_gemm_tn_pair<256, pnm::MODE_AUX>(c, g_num_sms, g_err_ptr, st);
    if (Z) return pnm::launch_gemm_tn_pair<256, pnm::MODE_Z>(c, g_num_sms, g_err_ptr, st);
    return pnm::launch_gemm_tn_pair<256, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
  }
  if (AUX) return pnm::launch_gemm_tn<128, pnm::MODE_AUX>(c, g_num_sms, g_err_ptr, st);
  if (Z) return pnm::launch_gemm_tn<128, pnm::MODE_Z>(c, g_num_sms, g_err_ptr, st);
  if (bn == 0) {
    bn = (N > 128) ? 256 : 128;
    // N <= 128 with many row tiles: 256-row x 128-column tiles of the BN = 256 instantiation (B read once per 256 rows)
    if (bn == 128 && N > 64 && (long long)M >= 256LL * 2 * g_num_sms) { bn = 256; c.split_m = 1; }
  } else if (bn == -256) { bn = 256; c.split_m = 1; }
  if (bn == 256) return pnm::launch_gemm_tn<256, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
  return pnm::launch_gemm_tn<128, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
}


// `batch` problems of the same shape in one launch: A [batch * Mp, K] (Mp % 128 == 0, problem b in rows b Mp ..), B [batch * N, K],
// C / AUX [batch * Mp, N], bias [batch * N] or null; C_b = epilogue(A_b @ B_b^T).  Rows that pad a problem to Mp are computed
// like any other (their inputs should be finite).
int pnm_gemm_tn_stacked(const void* A, int lda, const void* B, int ldb, void* C, int ldc, const void* AUX, int ldaux, int Mp, int N,
                        int K, int batch, const float* bias, int act, int aux_mode, int max_ctas, void* stream) {
  if (ensure_init()) return -1;
  if (Mp <= 0 || N <= 0 || K <= 0 || batch <= 0 || (Mp % 128)) return -2;
  if ((N % 8) || (K % 8) || (lda % 8) || (ldb % 8) || (ldc % 8)) return -3;
  if ((aux_mode != 0) != (AUX != nullptr)) return -6;
  if (act == pnm::ACT_SOFTMAX64) return -7;
  pnm::GemmCall c;
  c.A = A; c.lda = lda; c.A2 = nullptr; c.lda2 = 0; c.A3 = nullptr; c.lda3 = 0; c.B = B; c.ldb = ldb; c.C = C; c.ldc = ldc;
  c.Z = nullptr; c.ldz = 0; c.AUX = AUX; c.ldaux = ldaux;
  c.M = Mp * batch; c.N = N; c.K = K; c.K1 = K; c.K2 = K;
  c.bias = bias; c.scale = nullptr; c.group_out = nullptr;
  c.act = act; c.aux_mode = aux_mode; c.scale_post = 0; c.max_ctas = max_ctas;
  c.batch = batch;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (AUX) return pnm::launch_gemm_tn<128, pnm::MODE_AUX>(c, g_num_sms, g_err_ptr, st);
  if (N > 128) return pnm::launch_gemm_tn<256, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
  return pnm::launch_gemm_tn<128, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
}

// y[n, h, w, :] = act(sum over taps and input channels of x[n, h + dy, w + dx, :] W[:, tap, :] + bias): stride-1 "same"
// convolution of a channels-last bf16 image on the tensor cores.  weight: [cout, ksize*ksize*cin] bf16, tap-major
// (tap = ky * ksize + kx).  Requires cin % 64 == 0, cout % 8 == 0, odd ksize.
int pnm_conv2d_nhwc(const void* x, const void* weight, void* y, int n, int h, int w, int cin, int cout, int ksize,
                    const float* bias, int act, int bn, int max_ctas, void* stream) {
  if (ensure_init()) return -1;
  if (n <= 0 || h <= 0 || w <= 0 || cin <= 0 || cout <= 0) return -2;
  if ((cin % 64) || (cout % 8) || !(ksize & 1) || ksize < 1 || ksize > 7) return -3;
  pnm::GemmCall c{};
  c.A = x; c.lda = cin; c.A2 = nullptr; c.lda2 = 0; c.A3 = nullptr; c.lda3 = 0;
  c.B = weight; c.ldb = ksize * ksize * cin; c.C = y; c.ldc = cout; c.Z = nullptr; c.ldz = 0; c.AUX = nullptr; c.ldaux = 0;
  c.M = n * h * w; c.N = cout; c.K = ksize * ksize * cin; c.K1 = c.K; c.K2 = c.K;
  c.bias = bias; c.scale = nullptr; c.group_out = nullptr; c.act = act; c.aux_mode = 0; c.scale_post = 0;
  c.max_ctas = max_ctas;
  c.conv = 1; c.img_n = n; c.img_h = h; c.img_w = w; c.cin = cin; c.ksize = ksize;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0 && pair_gemm_enabled() && pnm::pair_gemm_applicable(c)) {
    if (cout > 128) return pnm::launch_gemm_tn_pair<256, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
    return pnm::launch_gemm_tn_pair<128, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
  }
  if (bn == 0) {
    bn = (cout > 128) ? 256 : 128;
    if (bn == 128 && cout > 64 && (long long)n * h * w >= 256LL * 2 * g_num_sms) { bn = 256; c.split_m = 1; }
  } else if (bn == -256) { bn = 256; c.split_m = 1; }
  if (bn == 256) return pnm::launch_gemm_tn<256, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
  return pnm::launch_gemm_tn<128, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
}

namespace pnm {
// Copies the first and the last image row of every image of x [n, h, w, c] (bf16) into this rank's mailbox, then raises
// the flags in the neighbours' buffers: the block that finishes last does the two release stores.
__global__ void __launch_bounds__(256) halo_publish_kernel(const uint4* __restrict__ x, uint4* __restrict__ top, uint4* __restrict__ bottom,
                                                          int n, int h, long long row_vecs /* w*c/8 */, uint32_t* flag_at_up,
                                                          uint32_t* flag_at_down, uint32_t epoch, unsigned int* counter) {
  const long long total = 2LL * n * row_vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int side = (int)(i / (n * row_vecs));
    const long long r = i - side * n * row_vecs;
    const long long img = r / row_vecs, v = r - img * row_vecs;
    const uint4 val = x[(img * h + (side ? h - 1 : 0)) * row_vecs + v];
    (side ? bottom : top)[img * row_vecs + v] = val;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {
      *counter = 0;
      __threadfence_system();
      if (flag_at_up) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag_at_up), "r"(epoch) : "memory");
      if (flag_at_down) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag_at_down), "r"(epoch) : "memory");
    }
  }
}
}  // namespace pnm

// Publish the boundary rows of a height slab for the neighbours' halo reads.  top / bottom: this rank's mailbox blocks
// [n, 1, w, c]; flag_at_up / flag_at_down: peer-mapped addresses of the flags the neighbours wait on (null at the edges).
int pnm_halo_publish(const void* x, void* top, void* bottom, int n, int h, int w, int c, void* flag_at_up, void* flag_at_down,
                     unsigned int epoch, void* counter, void* stream) {
  if (ensure_init()) return -1;
  if (n <= 0 || h <= 0 || ((long long)w * c) % 8) return -2;
  const long long row_vecs = (long long)w * c / 8, total = 2LL * n * row_vecs;
  const unsigned grid = (unsigned)std::min<long long>((total + 255) / 256, 4 * g_num_sms);
  pnm::halo_publish_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), reinterpret_cast<uint4*>(top), reinterpret_cast<uint4*>(bottom), n, h, row_vecs,
      reinterpret_cast<uint32_t*>(flag_at_up), reinterpret_cast<uint32_t*>(flag_at_down), epoch,
      reinterpret_cast<unsigned int*>(counter));
  return cudaGetLastError() == cudaSuccess ? 0 : -52;
}

// pnm_conv2d_nhwc for a height slab: the rows above / below come from the neighbours' published rows (up_rows / down_rows,
// peer-mapped, null at the outer edges) once flag_up / flag_down (local memory) carry `epoch`.  3 x 3 only, h % 8 == 0.
int pnm_conv2d_nhwc_halo(const void* x, const void* weight, void* y, int n, int h, int w, int cin, int cout, const float* bias,
                         int act, const void* up_rows, const void* down_rows, const void* flag_up, const void* flag_down,
                         unsigned int epoch, int bn, int max_ctas, void* stream, double budget_s) {
  if (ensure_init()) return -1;
  if (n <= 0 || h <= 0 || w <= 0 || (cin % 64) || (cout % 8) || (h % 8)) return -3;
  pnm::GemmCall c{};
  c.A = x; c.lda = cin; c.B = weight; c.ldb = 9 * cin; c.C = y; c.ldc = cout;
  c.M = n * h * w; c.N = cout; c.K = 9 * cin; c.K1 = c.K; c.K2 = c.K;
  c.bias = bias; c.act = act; c.max_ctas = max_ctas;
  c.conv = 1; c.img_n = n; c.img_h = h; c.img_w = w; c.cin = cin; c.ksize = 3;
  c.halo = 1; c.up_rows = up_rows; c.down_rows = down_rows;
  c.flag_up = reinterpret_cast<const uint32_t*>(flag_up); c.flag_down = reinterpret_cast<const uint32_t*>(flag_down);
  c.halo_epoch = epoch; c.halo_budget_s = budget_s;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 0 && pair_gemm_enabled() && pnm::pair_gemm_applicable(c)) {
    if (cout > 128) return pnm::launch_gemm_tn_pair<256, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
    return pnm::launch_gemm_tn_pair<128, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
  }
  if (bn == 0) {
    bn = (cout > 128) ? 256 : 128;
    if (bn == 128 && cout > 64 && (long long)n * h * w >= 256LL * 2 * g_num_sms) { bn = 256; c.split_m = 1; }
  } else if (bn == -256) { bn = 256; c.split_m = 1; }
  if (bn == 256) return pnm::launch_gemm_tn<256, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
  return pnm::launch_gemm_tn<128, pnm::MODE_PLAIN>(c, g_num_sms, g_err_ptr, st);
}

int pnm_gemm_nt(const void* A, int lda, const void* B, int ldb, float* out, int ldo, float* colsum, int M, int Na,
                int Nb, int max_ctas, void* stream) {
  if (ensure_init()) return -1;
  if (M <= 0 || Na <= 0 || Nb <= 0) return -2;
  if ((Na % 8) || (Nb % 8) || (lda % 8) || (ldb % 8)) return -3;
  pnm::NtCall c;
  c.A = A; c.lda = lda; c.B = B; c.ldb = ldb; c.out = out; c.ldo = ldo; c.colsum = colsum;
  c.M = M; c.Na = Na; c.Nb = Nb; c.max_ctas = max_ctas;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pair_gemm_enabled() && pnm::pair_gemm_nt_applicable(c)) {
    if (Nb > 128) return pnm::launch_gemm_nt_pair<256>(c, g_num_sms, g_err_ptr, st);
    return pnm::launch_gemm_nt_pair<128>(c, g_num_sms, g_err_ptr, st);
  }
  if (Nb > 128) return pnm::launch_gemm_nt<256>(c, g_num_sms, g_err_ptr, st);
  return pnm::launch_gemm_nt<128>(c, g_num_sms, g_err_ptr, st);
}

// `batch` weight-gradient problems in one launch: A [batch * Mp, Na], B [batch * Mp, Nb] (Mp % 64 == 0; rows that pad a problem
// must be zero in A or B), out [batch, Na, Nb] fp32 (accumulated into), colsum [batch, Na] or null.
int pnm_gemm_nt_stacked(const void* A, int lda, const void* B, int ldb, float* out, float* colsum, int Mp, int Na, int Nb, int batch,
                        int max_ctas, void* stream) {
  if (ensure_init()) return -1;
  if (Mp <= 0 || Na <= 0 || Nb <= 0 || batch <= 0 || (Mp % 64)) return -2;
  if ((Na % 8) || (Nb % 8) || (lda % 8) || (ldb % 8)) return -3;
  pnm::NtCall c;
  c.A = A; c.lda = lda; c.B = B; c.ldb = ldb; c.out = out; c.ldo = Nb; c.colsum = colsum;
  c.M = Mp * batch; c.Na = Na; c.Nb = Nb; c.max_ctas = max_ctas;
  c.batch = batch; c.out_stride = (long long)Na * Nb;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (Nb > 128) return pnm::launch_gemm_nt<256>(c, g_num_sms, g_err_ptr, st);
  return pnm::launch_gemm_nt<128>(c, g_num_sms, g_err_ptr, st);
}

// dW[cout, 9 * cin] (fp32, tap-major, accumulated into `out`) = sum over pixels of dy[pixel, :]^T x[pixel + tap, :] for a 3 x 3
// stride-1 "same" convolution of channels-last bf16 tensors; colsum (optional) accumulates the bias gradient.
// up_rows / down_rows (optional, [n, 1, w, cin]): the input rows just above / below a height slab; when flag_up /
// flag_down are given the kernel first waits (bounded) until they carry `epoch`.  cin % 64 == 0, cout >= 64, cout % 8 == 0.
int pnm_conv2d_wgrad_nhwc(const void* dy, const void* x, float* out, float* colsum, int n, int h, int w, int cin, int cout,
                          const void* up_rows, const void* down_rows, const void* flag_up, const void* flag_down,
                          unsigned int epoch, double budget_s, int max_ctas, void* stream) {
  if (ensure_init()) return -1;
  if (n <= 0 || h <= 0 || w <= 0 || (cin % 64) || (cout % 8) || cout < 64) return -3;
  pnm::NtCall c{};
  c.A = dy; c.lda = cout; c.B = x; c.ldb = cin; c.out = out; c.ldo = 9 * cin; c.colsum = colsum;
  c.M = 0; c.Na = cout; c.Nb = 9 * cin; c.max_ctas = max_ctas;
  c.conv = 1; c.img_n = n; c.img_h = h; c.img_w = w; c.cin = cin;
  c.halo = (up_rows || down_rows) ? 1 : 0;
  c.up_rows = up_rows; c.down_rows = down_rows;
  c.flag_up = reinterpret_cast<const uint32_t*>(flag_up); c.flag_down = reinterpret_cast<const uint32_t*>(flag_down);
  c.halo_epoch = epoch; c.halo_budget_s = budget_s;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pair_gemm_enabled() && pnm::pair_gemm_nt_applicable(c)) {
    if ((9 * cin) % 256 == 0) return pnm::launch_gemm_nt_pair<256>(c, g_num_sms, g_err_ptr, st);
    return pnm::launch_gemm_nt_pair<128>(c, g_num_sms, g_err_ptr, st);
  }
  if ((9 * cin) % 256 == 0) return pnm::launch_gemm_nt<256>(c, g_num_sms, g_err_ptr, st);
  return pnm::launch_gemm_nt<128>(c, g_num_sms, g_err_ptr, st);
}

int pnm_layernorm_fwd(const void* x, const void* r, const float* gamma, const float* beta, void* y, void* sum_out,
                      float* mean, float* rstd, const void* post, long long M, int C, float eps, void* stream) {
  if (ensure_init()) return -1;
  return pnm::launch_layernorm_fwd(x, r, gamma, beta, y, sum_out, mean, rstd, post, M, C, eps, g_num_sms,
                                   reinterpret_cast<cudaStream_t>(stream));
}

long long pnm_layernorm_bwd_scratch_floats(long long M, int C) {
  if (ensure_init()) return -1;
  return (long long)pnm::layernorm_bwd_grid(M, g_num_sms) * 2 * C;
}

int pnm_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                      const void* dres, void* dx, float* dgamma, float* dbeta, float* scratch, long long M, int C,
                      void* stream) {
  if (ensure_init()) return -1;
  return pnm::launch_layernorm_bwd(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, scratch, M, C, g_num_sms,
                                   reinterpret_cast<cudaStream_t>(stream));
}

int pnm_gather_rows(const void* in, int ldi, const int* idx, const float* scale, void* out, int ldo, long long E,
                    int C, void* stream) {
  if (ensure_init()) return -1;
  return pnm::launch_gather_rows(in, ldi, idx, scale, out, ldo, E, C, g_num_sms, reinterpret_cast<cudaStream_t>(stream));
}

int pnm_segment_sum(const void* in, int ldi, const int* perm, const int* offsets, void* out, int ldo, long long N,
                    int C, int accumulate, int mode, void* stream) {
  if (ensure_init()) return -1;
  return pnm::launch_segment_sum(in, ldi, perm, offsets, out, ldo, N, C, accumulate, mode, g_num_sms,
                                 reinterpret_cast<cudaStream_t>(stream));
}

// bases: host array of `world` peer-mapped pointers to the symmetric buffers (this rank's own included).
int pnm_peer_allreduce(const float* in, float* out, long long n, float scale, int two_shot, const void* const* bases,
                       int rank, int world, unsigned int epoch, long long capacity_floats, double budget_s,
                       void* stream, const void* epoch_base, int max_ctas) {
  if (ensure_init()) return -1;
  if (world > pnm::kPeerMaxRanks || world < 1) return -50;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  return pnm::launch_peer_allreduce(in, out, n, scale, two_shot, p, max_ctas, g_err_ptr, reinterpret_cast<cudaStream_t>(stream));
}

int pnm_peer_allreduce_bf16(float* io, long long n, float scale, const void* const* bases, int rank, int world,
                            unsigned int epoch, long long capacity_floats, double budget_s, void* stream,
                            const void* epoch_base, int max_ctas) {
  if (ensure_init()) return -1;
  if (world > pnm::kPeerMaxRanks || world < 1) return -50;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  return pnm::launch_peer_allreduce_bf16(io, n, scale, p, max_ctas, g_err_ptr, reinterpret_cast<cudaStream_t>(stream));
}

int pnm_peer_signal(const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats,
                    void* stream, const void* epoch_base) {
  if (ensure_init()) return -1;
  if (world > pnm::kPeerMaxRanks || world < 1) return -50;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, 1.0, epoch_base);
  pnm::peer_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -51;
}

int pnm_peer_pull(const void* src, void* dst, long long bytes, int flag_from, const void* const* bases, int rank, int world,
                  unsigned int epoch, long long capacity_floats, double budget_s, void* stream, const void* epoch_base,
                  int max_ctas) {
  if (ensure_init()) return -1;
  if (world > pnm::kPeerMaxRanks || world < 1) return -50;
  if (bytes <= 0) return 0;
  if ((bytes & 15) || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return -53;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  const long long nvec = bytes / 16;
  int grid = (int)std::min<long long>((nvec + 2047) / 2048, max_ctas > 0 ? max_ctas : 64);
  if (grid < 1) grid = 1;
  pnm::peer_pull_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), reinterpret_cast<uint4*>(dst), nvec, p, flag_from, g_err_ptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -51;
}

int pnm_peer_pull_reduce(float* dst, long long block, const void* const* bases, int rank, int world, unsigned int epoch,
                         long long capacity_floats, double budget_s, void* stream, const void* epoch_base, int max_ctas) {
  if (ensure_init()) return -1;
  if (world > pnm::kPeerMaxRanks || world < 1) return -50;
  if (block <= 0) return 0;
  if ((block & 3) || block * world > capacity_floats || (reinterpret_cast<uintptr_t>(dst) & 15)) return -53;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  int grid = (int)std::min<long long>((block / 4 + 511) / 512, max_ctas > 0 ? max_ctas : 96);
  if (grid < 1) grid = 1;
  pnm::peer_pull_reduce_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dst, block, p, g_err_ptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -51;
}

// dst[i] = sum_r srcs[r][i] (srcs: host array of 8 peer-mapped addresses, unused entries repeating a valid one), n % 4 == 0.
int pnm_peer_sum_blocks(float* dst, const void* const* srcs, long long n, int wait, const void* const* bases, int rank, int world,
                        unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base, void* stream,
                        int max_ctas) {
  if (ensure_init()) return -1;
  if (world > pnm::kPeerMaxRanks || world < 1) return -50;
  if (n <= 0) return 0;
  if ((n & 3) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -53;
  pnm::PeerSrcs ps;
  for (int r = 0; r < pnm::kPeerMaxRanks; ++r) {
    if (reinterpret_cast<uintptr_t>(srcs[r]) & 15) return -53;
    ps.p[r] = reinterpret_cast<const float*>(srcs[r]);
  }
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  int grid = (int)std::min<long long>((n / 4 + 511) / 512, max_ctas > 0 ? max_ctas : 2 * g_num_sms);
  if (grid < 1) grid = 1;
  pnm::peer_sum_blocks_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dst, ps, n, wait, p, g_err_ptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -51;
}

// Non-blocking read of the error word: enqueues a copy into pinned host memory on `stream`.
int pnm_error_copy_async(int* pinned_host, void* stream) {
  if (ensure_init()) return -1;
  return cudaMemcpyAsync(pinned_host, g_err_ptr, sizeof(int), cudaMemcpyDeviceToHost, reinterpret_cast<cudaStream_t>(stream)) ==
                 cudaSuccess ? 0 : -1;
}

int pnm_peer_flag_bytes() { return pnm::kFlagBytes; }

// Launch a wait on `flag` that gives up after budget_s seconds; *status_out = 1 if satisfied, 0 if it timed out.
int pnm_peer_wait_probe(const void* flag, unsigned int expect, double budget_s, int* status_out, void* stream) {
  if (ensure_init()) return -1;
  pnm::peer_wait_probe_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint32_t*>(flag), expect, (unsigned long long)(budget_s * 1e9), g_err_ptr, status_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -52;
}

int pnm_flash_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int BH, int Sq, int Skv, int D,
                       int ldv, float scale, int causal, int v_transposed, int p_in_tmem, void* stream) {
  if (ensure_init()) return -1;
  if (!q || !k || !v || !out || BH <= 0 || Sq <= 0 || Skv <= 0 || !(scale > 0.f)) return -1;
  if (v_transposed && (ldv < Skv || (ldv & 7))) return -1;
  pnm::FlashCall c{q, k, v, out, lse, BH, Sq, Skv, ldv, scale, causal};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int variant = (D == 128 ? 4 : 0) | (v_transposed ? 2 : 0) | (p_in_tmem ? 1 : 0);
  if (D != 64 && D != 128) return -1;
  switch (variant) {
    case 0: return pnm::launch_flash_fwd<64, false, false>(c, g_err_ptr, st);
    case 1: return pnm::launch_flash_fwd<64, false, true>(c, g_err_ptr, st);
    case 2: return pnm::launch_flash_fwd<64, true, false>(c, g_err_ptr, st);
    case 3: return pnm::launch_flash_fwd<64, true, true>(c, g_err_ptr, st);
    case 4: return pnm::launch_flash_fwd<128, false, false>(c, g_err_ptr, st);
    case 5: return pnm::launch_flash_fwd<128, false, true>(c, g_err_ptr, st);
    case 6: return pnm::launch_flash_fwd<128, true, false>(c, g_err_ptr, st);
    default: return pnm::launch_flash_fwd<128, true, true>(c, g_err_ptr, st);
  }
}

}  // extern "C"
