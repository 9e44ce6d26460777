// Declarations shared by the translation units of the kernel library (not part of the C ABI).
#pragma once
#include "peer.cuh"

namespace pnm {

constexpr int kMaxDevices = 64;

int current_device();          // index of the current CUDA device (0 when it cannot be read)
int* error_word_ptr();         // device address of the library's error word on the current device (null on failure)
int num_sms();                 // SM count of the current device
PeerArgs make_peer_args(const void* const* bases, int rank, int world, unsigned int epoch, long long capacity_floats,
                        double budget_s, const void* epoch_base);

// Set-once-per-device bookkeeping for cudaFuncSetAttribute calls: returns true when `mask` did not yet carry the
// bit of the current device (and sets it).
inline bool first_use_on_device(unsigned long long& mask) {
  const int dev = current_device();
  const unsigned long long bit = 1ull << (dev & 63);
  if (mask & bit) return false;
  mask |= bit;
  return true;
}

}  // namespace pnm
