// Partitioned-graph halo exchange fused into the message-passing gathers (bf16 feature rows).
//
// A graph is partitioned by destination node: every rank owns a contiguous block of nodes and all edges that end in
// them.  The source of an edge may be a node of another rank (a "halo" node).  The reference moves halo features
// with an indexed all-to-all-v before the edge block and the reverse + index_add_ in backward
// (physicsnemo/distributed/utils.py:541-707).  Here:
//
//   halo_publish   gathers this rank's boundary rows (the rows some peer needs) into a compact mailbox in symmetric
//                  memory; the block that finishes last raises one flag per peer;
//   gather_halo    the edge gather itself: out[e] = local row, or -- for a halo source -- the row read straight from
//                  the owner's mailbox over NVLink, after a bounded wait on the flags in the kernel's prologue;
//   halo_pull_add  backward: every rank has left the gradient rows of ITS halo nodes in its own mailbox; the owner of
//                  a boundary row adds up the copies of all peers that use it (direct peer loads, fixed order, no
//                  atomics) and accumulates them into its local gradient.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "pnm_api.h"
#include "pnm_internal.h"

namespace pnm {

struct MailboxPtrs { const __nv_bfloat16* p[kPeerMaxRanks]; };

__global__ void __launch_bounds__(256)
graph_halo_publish_kernel(const __nv_bfloat16* __restrict__ in, int ldi, const int* __restrict__ send_idx,
                    __nv_bfloat16* __restrict__ mailbox, long long n_send, int C, PeerArgs peer, unsigned int* counter) {
  const int cpr = C >> 3;
  const long long total = n_send * cpr;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / cpr;
    const int c = int(t - r * cpr) << 3;
    const long long src = send_idx ? (long long)__ldg(send_idx + r) : r;
    *reinterpret_cast<uint4*>(mailbox + r * C + c) = *reinterpret_cast<const uint4*>(in + src * ldi + c);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(counter, 1u) == gridDim.x - 1) {
    *counter = 0;
    peer_small_publish(peer, peer_epoch(peer));
  }
}

// idx[e] < n_local: local row; else halo h = idx[e] - n_local lives in mailbox row halo_slot[h] of rank halo_owner[h]
__global__ void __launch_bounds__(256)
gather_halo_kernel(const __nv_bfloat16* __restrict__ in, int ldi, const int* __restrict__ idx, int n_local,
                   const int* __restrict__ halo_owner, const int* __restrict__ halo_slot, MailboxPtrs mb,
                   __nv_bfloat16* __restrict__ out, int ldo, long long E, int C, PeerArgs peer, int wait, int* err) {
  __shared__ int sh_ok;
  bool ok = true;
  if (wait) ok = peer_small_wait(peer, peer_epoch(peer), err, &sh_ok);
  const int cpr = C >> 3;
  const long long total = E * cpr;
  const uint4 nan4 = make_uint4(0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u, 0x7fc07fc0u);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long e = t / cpr;
    const int c = int(t - e * cpr) << 3;
    const int src = __ldg(idx + e);
    uint4 v;
    if (src < n_local) v = *reinterpret_cast<const uint4*>(in + (long long)src * ldi + c);
    else if (!ok) v = nan4;
    else {
      const int h = src - n_local;
      v = __ldcg(reinterpret_cast<const uint4*>(mb.p[__ldg(halo_owner + h)] + (long long)__ldg(halo_slot + h) * C + c));
    }
    *reinterpret_cast<uint4*>(out + e * (long long)ldo + c) = v;
  }
}

// boundary row b (local node bnd_row[b]) += sum over entries k in [bnd_off[b], bnd_off[b+1]) of mailbox[ent_peer[k]][ent_slot[k]]
__global__ void __launch_bounds__(256)
halo_pull_add_kernel(__nv_bfloat16* __restrict__ dn, int ldn, const int* __restrict__ bnd_row, const int* __restrict__ bnd_off,
                     const int* __restrict__ ent_peer, const int* __restrict__ ent_slot, MailboxPtrs mb, long long n_bnd, int C,
                     PeerArgs peer, int wait, int* err) {
  __shared__ int sh_ok;
  bool ok = true;
  if (wait) ok = peer_small_wait(peer, peer_epoch(peer), err, &sh_ok);
  const int cpr = C >> 3;
  const long long total = n_bnd * cpr;
  const float nanv = __int_as_float(0x7fc00000);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long b = t / cpr;
    const int c = int(t - b * cpr) << 3;
    __nv_bfloat16* dst = dn + (long long)__ldg(bnd_row + b) * ldn + c;
    const uint4 o = *reinterpret_cast<const uint4*>(dst);
    float acc[8];
    float2 f;
    f = unpack_bf16x2(o.x); acc[0] = f.x; acc[1] = f.y;
    f = unpack_bf16x2(o.y); acc[2] = f.x; acc[3] = f.y;
    f = unpack_bf16x2(o.z); acc[4] = f.x; acc[5] = f.y;
    f = unpack_bf16x2(o.w); acc[6] = f.x; acc[7] = f.y;
    for (int k = __ldg(bnd_off + b); k < __ldg(bnd_off + b + 1); ++k) {
      if (!ok) { for (int j = 0; j < 8; ++j) acc[j] = nanv; break; }
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(mb.p[__ldg(ent_peer + k)] + (long long)__ldg(ent_slot + k) * C + c));
      f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
      f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
      f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
      f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
    }
    uint4 w;
    w.x = pack_bf16x2(acc[0], acc[1]); w.y = pack_bf16x2(acc[2], acc[3]);
    w.z = pack_bf16x2(acc[4], acc[5]); w.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(dst) = w;
  }
}

// ptrs: host array of kPeerMaxRanks entries (unused ones repeat a valid address)
static MailboxPtrs make_mb(const void* const* ptrs) {
  MailboxPtrs m;
  for (int r = 0; r < kPeerMaxRanks; ++r) m.p[r] = reinterpret_cast<const __nv_bfloat16*>(ptrs[r]);
  return m;
}

static int grid_rows(long long items, int sms) {
  long long want = (items + 255) / 256, cap = (long long)sms * 16;
  int g = (int)(want < cap ? want : cap);
  return g < 1 ? 1 : g;
}

}  // namespace pnm

extern "C" {

// Copy rows send_idx[0 .. n_send) of `in` into this rank's mailbox and raise the flags of call `epoch` on every peer
// (peer arguments as in pnm_peer_allreduce).  counter: zeroed device uint32 (reset by the kernel).  n_send may be 0.
int pnm_graph_halo_publish(const void* in, int ldi, const int* send_idx, void* mailbox, long long n_send, int C,
                           const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats,
                           const void* epoch_base, void* counter, void* stream) {
  if (C % 8 || ldi % 8 || world < 1 || world > pnm::kPeerMaxRanks || !counter) return -2;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, 1.0, epoch_base);
  const int grid = n_send > 0 ? pnm::grid_rows(n_send * (C >> 3), pnm::num_sms()) : 1;
  pnm::graph_halo_publish_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)in, ldi, send_idx, (__nv_bfloat16*)mailbox,
                                                                   n_send, C, p, (unsigned int*)counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// out[e, :] = in[idx[e], :] for idx[e] < n_local, else the halo row from its owner's mailbox (mailboxes: host array of
// 8 peer-mapped mailbox addresses, rank order, unused entries repeating a valid one).  wait != 0: first wait for every rank's flag of call `epoch`.
int pnm_graph_gather_halo(const void* in, int ldi, const int* idx, int n_local, const int* halo_owner, const int* halo_slot,
                          const void* const* mailboxes, void* out, int ldo, long long E, int C, int wait,
                          const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats,
                          double budget_s, const void* epoch_base, void* stream) {
  if (C % 8 || ldi % 8 || ldo % 8 || world < 1 || world > pnm::kPeerMaxRanks) return -2;
  if (E <= 0) return 0;
  int* err = pnm::error_word_ptr();
  if (!err) return -1;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  pnm::gather_halo_kernel<<<pnm::grid_rows(E * (C >> 3), pnm::num_sms()), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)in, ldi, idx, n_local, halo_owner, halo_slot, pnm::make_mb(mailboxes), (__nv_bfloat16*)out, ldo, E,
      C, p, wait, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dn[bnd_row[b], :] += sum of the peers' mailbox rows listed for boundary row b (CSR bnd_off / ent_peer / ent_slot).
int pnm_graph_halo_pull_add(void* dn, int ldn, const int* bnd_row, const int* bnd_off, const int* ent_peer, const int* ent_slot,
                            const void* const* mailboxes, long long n_bnd, int C, int wait, const void* const* bases, int rank,
                            int world, unsigned int epoch, long long capacity_floats, double budget_s, const void* epoch_base,
                            void* stream) {
  if (C % 8 || ldn % 8 || world < 1 || world > pnm::kPeerMaxRanks) return -2;
  int* err = pnm::error_word_ptr();
  if (!err) return -1;
  const pnm::PeerArgs p = pnm::make_peer_args(bases, rank, world, epoch, capacity_floats, budget_s, epoch_base);
  const int grid = n_bnd > 0 ? pnm::grid_rows(n_bnd * (C >> 3), pnm::num_sms()) : 1;
  pnm::halo_pull_add_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)dn, ldn, bnd_row, bnd_off, ent_peer, ent_slot,
                                                                    pnm::make_mb(mailboxes), n_bnd, C, p, wait, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
