// Symmetric peer-memory state shared by the collective kernels and by the kernels that fuse a collective into
// their epilogue / prologue (GEMM push, fold + add + RMSNorm + quantise).  Layout of every rank's region:
//     [ 2 parities ][ W source slots ][ slot_bytes ]   payload pushed by the source rank
//     [ 2 parities ][ W source slots ][ kCommMaxCtas ] uint32 flags (epoch numbers), one per pushed slice / tile
//     pick table: [ 2 parities ][ W ][ kPickRows ] (value, id) pairs + [2][W] flags
// Peer memory is only touched with plain vector stores, volatile loads and system-scope flag accesses.
#pragma once
#include <stdint.h>

#include "common/common.h"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kCommMaxWorld = 8;
constexpr int kCommMaxCtas = 64;
constexpr int kPickRows = 256;

struct CommState {
  unsigned char* peers[kCommMaxWorld];  // base of every rank's symmetric region (peer-mapped pointers)
  int world, rank;
  size_t slot_bytes;
  uint32_t* epoch;      // device counter of completed all-reduces (local memory)
  uint32_t* done_ctas;  // CTAs finished in the current call (local)
  uint32_t* pick_epoch;
};

__device__ __forceinline__ unsigned char* payload(const CommState& c, int owner, int parity, int src) {
  return c.peers[owner] + (static_cast<size_t>(parity) * c.world + src) * c.slot_bytes;
}
__device__ __forceinline__ uint32_t* flag(const CommState& c, int owner, int parity, int src, int cta) {
  unsigned char* base = c.peers[owner] + 2 * static_cast<size_t>(c.world) * c.slot_bytes;
  return reinterpret_cast<uint32_t*>(base) + (static_cast<size_t>(parity) * c.world + src) * kCommMaxCtas + cta;
}
__device__ __forceinline__ unsigned char* pick_base(const CommState& c, int owner) {
  return c.peers[owner] + 2 * static_cast<size_t>(c.world) * c.slot_bytes +
         2 * static_cast<size_t>(c.world) * kCommMaxCtas * sizeof(uint32_t);
}

// Bounded spin on a flag written by a peer; false when it gave up (about 2 s).
__device__ __forceinline__ bool wait_flag(const uint32_t* f, uint32_t want) {
  for (int i = 0; i < 1 << 14; ++i)
    if (ld_acquire_sys(f) == want) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 256; ++i) {
      if (ld_acquire_sys(f) == want) return true;
      __nanosleep(64);
    }
    if (clock64() - t0 > 4000000000ll) return false;
  }
}

}  // namespace dgpp

// Host-side handle returned by dgpp_comm_create.
struct DgppComm {
  dgpp::CommState st;
  void* local;
  void* opened[dgpp::kCommMaxWorld];
  size_t region_bytes;
};
