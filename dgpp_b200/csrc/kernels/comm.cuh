// Symmetric peer-memory state shared by the collective kernels and by the kernels that fuse a collective into
// their epilogue / prologue (GEMM push, fold + add + RMSNorm + quantise).  Layout of every rank's region:
//     [ 2 parities ][ W source slots ][ slot_bytes ]   payload pushed by the source rank
//     [ 2 parities ][ W source slots ][ kCommMaxCtas ] uint32 flags (epoch numbers), one per pushed slice / tile
//     pick table: [ 2 parities ][ W ][ kPickRows ] (value, id) pairs + [2][W] flags
//     reduce-scatter tables: [ 2 parities ][ W source ranks ][ kCommMaxCtas token tiles ] uint32 arrival counters
//                            (how many output tiles of that token tile the source has pushed; the owner zeroes them
//                            after folding), [ 2 parities ][ kCommMaxCtas ][ kRsMaxChunks ] uint32 all-gather flags
//                            (epoch numbers), [ kCommMaxCtas ] uint32 local fold counters
// Peer memory is only touched with plain vector stores, volatile loads and system-scope flag accesses.
#pragma once
#include <stdint.h>

#include "common/common.h"
#include "common/ptx.cuh"

namespace dgpp {

constexpr int kCommMaxWorld = 8;
constexpr int kCommMaxCtas = 64;
constexpr int kPickRows = 256;
constexpr int kRsMaxChunks = 16;

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

__device__ __forceinline__ unsigned char* rs_base(const CommState& c, int owner) {
  const size_t off = 2 * static_cast<size_t>(c.world) * kPickRows * 8 + 2 * static_cast<size_t>(c.world) * sizeof(uint32_t);
  return pick_base(c, owner) + ((off + 255) & ~static_cast<size_t>(255));
}
// Arrival counter of (source rank, token tile) in `owner`'s region.
__device__ __forceinline__ uint32_t* rs_counter(const CommState& c, int owner, int parity, int src, int tile) {
  return reinterpret_cast<uint32_t*>(rs_base(c, owner)) + (static_cast<size_t>(parity) * c.world + src) * kCommMaxCtas + tile;
}
// All-gather flag of (token tile, column chunk) in `owner`'s region, written by the tile's owner rank.
__device__ __forceinline__ uint32_t* ag_flag(const CommState& c, int owner, int parity, int tile, int chunk) {
  uint32_t* base = reinterpret_cast<uint32_t*>(rs_base(c, owner)) + 2 * static_cast<size_t>(c.world) * kCommMaxCtas;
  return base + (static_cast<size_t>(parity) * kCommMaxCtas + tile) * kRsMaxChunks + chunk;
}
__device__ __forceinline__ uint32_t* rs_local_done(const CommState& c, int tile) {
  uint32_t* base = reinterpret_cast<uint32_t*>(rs_base(c, c.rank)) + 2 * static_cast<size_t>(c.world) * kCommMaxCtas +
                   2 * static_cast<size_t>(kCommMaxCtas) * kRsMaxChunks;
  return base + tile;
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
