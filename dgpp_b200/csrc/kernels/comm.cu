// Tensor-parallel collectives over NVLink peer memory, issued from our own kernels (no NCCL on this path).
//
// Symmetric memory: every rank cudaMallocs one region of the same size and shares it through CUDA IPC;
// each rank keeps a device table with the W peer base pointers (its own included).  Region layout:
//     [ 2 parities ][ W source slots ][ slot_bytes ]   payload pushed by the source rank
//     [ 2 parities ][ W source slots ][ kMaxCtas ]     uint32 flags (epoch numbers)
//     pick table: [ 2 parities ][ W ][ kPickRows ] (value, id) pairs + [2][W] flags
//
// One-shot all-reduce (decode sizes): every CTA owns a slice of the vector.  It stores its bf16 slice into
// slot `me` of every peer (plain 16-byte stores to peer pointers), fences at system scope, raises
// flag[parity][me][cta] = epoch on every peer with st.release.sys, then waits (ld.acquire.sys, bounded) for the
// W flags of its own slice and folds the W slices in ASCENDING RANK ORDER in fp32 with one bf16 rounding, so
// every rank computes bit-identical results.  Two parities are enough: a rank can enter all-reduce k + 2 only
// after every peer has pushed for k + 1, i.e. has finished reading k.
// The epoch lives in device memory and is advanced by the kernel itself, so a captured CUDA graph replays
// without any host-side arming.
// (reference behaviour: src/net/bus_kernel.cu:361,625,890 -- fold order and graph-node all-reduce; there the
//  transport is RoCE with host-pinned staging, here it is direct peer stores.)
#include <string.h>

#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/comm.cuh"

namespace dgpp {

// data: [n] bf16 (n multiple of 8), reduced in place.  resid (optional): out = bf16(resid + bf16(sum)).
__global__ void __launch_bounds__(256)
ar_oneshot_kernel(CommState c, bf16* __restrict__ data, const bf16* __restrict__ resid, int64_t n,
                  DeviceStatus* status) {
  pdl_wait();
  const uint32_t epoch = *c.epoch + 1;
  const int parity = epoch & 1;
  const int64_t nvec = n / 8;
  const int64_t per = (nvec + gridDim.x - 1) / gridDim.x;
  const int64_t v0 = blockIdx.x * per, v1 = min(nvec, v0 + per);
  // 1. push my slice to every rank (my own slot included: the fold below reads all W slots uniformly)
  for (int64_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
    const uint4 x = reinterpret_cast<const uint4*>(data)[v];
    for (int r = 0; r < c.world; ++r) {
      const int dst = (c.rank + r) % c.world;  // stagger destinations across ranks
      st_v4_global(payload(c, dst, parity, c.rank) + v * 16, x);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < c.world) st_release_sys(flag(c, threadIdx.x, parity, c.rank, blockIdx.x), epoch);
  // 2. wait for every source's flag of this slice
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag(c, c.rank, parity, threadIdx.x, blockIdx.x), epoch)) {
      if (atomicCAS(&status->code, 0, kTimeoutPeerFlag) == 0) status->detail = threadIdx.x;
      atomicAdd(&status->count, 1);
      ok_s = 0;
    }
  }
  __syncthreads();
  // 3. fold in ascending rank order
  if (ok_s) {
    for (int64_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int r = 0; r < c.world; ++r) {
        Pack16 p;
        p.u = ld_v4_global_volatile(payload(c, c.rank, parity, r) + v * 16);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += bf16_to_f32(p.h[j]);
      }
      Pack16 o;
      if (resid) {
        Pack16 rr;
        rr.u = reinterpret_cast<const uint4*>(resid)[v];
#pragma unroll
        for (int j = 0; j < 8; ++j) o.h[j] = f32_to_bf16(bf16_to_f32(rr.h[j]) + bf16_to_f32(f32_to_bf16(acc[j])));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o.h[j] = f32_to_bf16(acc[j]);
      }
      reinterpret_cast<uint4*>(data)[v] = o.u;
    }
  }
  // 4. the last CTA advances the epoch for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.done_ctas, 1u) == gridDim.x - 1) {
      *c.done_ctas = 0;
      *c.epoch = epoch;
      __threadfence();
    }
  }
}

// Vocab-sharded greedy pick: every rank contributes (value, id) of its slice per row; all ranks end up with
// the global winner (strictly greater value wins scanning ranks ascending => ties go to the lowest rank/id).
__global__ void __launch_bounds__(256)
pick_merge_kernel(CommState c, int32_t* __restrict__ ids, float* __restrict__ vals, int rows, DeviceStatus* status) {
  pdl_wait();
  const uint32_t epoch = *c.pick_epoch + 1;
  const int parity = epoch & 1;
  const int t = threadIdx.x;
  struct Pair { float v; int32_t i; };
  auto table = [&](int owner, int src) {
    return reinterpret_cast<Pair*>(pick_base(c, owner)) + (static_cast<size_t>(parity) * c.world + src) * kPickRows;
  };
  auto pflag = [&](int owner, int src) {
    return reinterpret_cast<uint32_t*>(pick_base(c, owner) + 2 * static_cast<size_t>(c.world) * kPickRows * sizeof(Pair)) +
           parity * c.world + src;
  };
  if (t < rows) {
    Pair p{vals[t], ids[t]};
    for (int r = 0; r < c.world; ++r) table(r, c.rank)[t] = p;
  }
  __threadfence_system();
  __syncthreads();
  if (t < c.world) st_release_sys(pflag(t, c.rank), epoch);
  __shared__ int ok_s;
  if (t == 0) ok_s = 1;
  __syncthreads();
  if (t < c.world && !wait_flag(pflag(c.rank, t), epoch)) {
    if (atomicCAS(&status->code, 0, kTimeoutPeerFlag) == 0) status->detail = 100 + t;
    atomicAdd(&status->count, 1);
    ok_s = 0;
  }
  __syncthreads();
  if (ok_s && t < rows) {
    float bv = -INFINITY;
    int32_t bi = 0;
    for (int r = 0; r < c.world; ++r) {
      const volatile Pair* q = table(c.rank, r) + t;
      const float v = q->v;
      const int32_t i = q->i;
      if (r == 0 || v > bv) { bv = v; bi = i; }
    }
    ids[t] = bi;
    vals[t] = bv;
  }
  __syncthreads();
  if (t == 0) *c.pick_epoch = epoch;
}

// Second half of a fused GEMM -> reduce-scatter -> all-gather (prefill sizes).  The tensor-parallel GEMM's epilogue
// has pushed every output tile [tile_rows tokens x 128 columns] as bf16 into slot `source rank` of the rank that OWNS
// those tokens (token tiles are dealt to ranks in contiguous runs of `tiles_per_rank`) and bumped the owner's arrival
// counter of (source, token tile).  Here CTA (token tile t, column chunk) of the owner waits until all W sources have
// delivered all `n_tiles` tiles of t, folds the W partial tiles in ascending rank order (fp32, one bf16 rounding),
// adds the residual stream, stores the new residual rows locally and into every peer's slot `owner` (those rows of a
// source slot are unused by the reduce-scatter), and raises the peers' all-gather flag of (t, chunk).  CTAs of tiles
// owned by other ranks wait for that flag and copy the rows into the local residual stream.  Blocks are numbered so
// that a rank's own (folding) tiles are scheduled first: a fold never waits on a copy, so the ranks cannot block
// each other.  Traffic per rank is 2 (W-1)/W of the tensor instead of (W-1) for the one-shot all-reduce.
// x: [T, H] bf16 residual stream, updated in place on every rank to bf16(x + bf16(sum over ranks of the partials)).
__global__ void __launch_bounds__(256)
rs_ag_kernel(CommState c, bf16* __restrict__ x, int T, int H, int tile_rows, int tiles_per_rank, int n_tiles,
             DeviceStatus* status) {
  pdl_wait();
  const uint32_t epoch = *c.epoch + 1;
  const int parity = epoch & 1;
  const int chunks = gridDim.y, chunk = blockIdx.y;
  const int tiles = gridDim.x;
  // own tiles first: block b of the grid's x dimension handles tile (first own tile + b) modulo the tile count
  const int own0 = min(c.rank * tiles_per_rank, tiles);
  const int t = (own0 + static_cast<int>(blockIdx.x)) % tiles;
  const int owner = min(t / tiles_per_rank, c.world - 1);
  const int r0 = t * tile_rows, rows = min(tile_rows, T - r0);
  const int cols = H / chunks, c0 = chunk * cols, vec = cols / 8;      // host checks H % (8 * chunks) == 0
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (owner == c.rank) {
    if (threadIdx.x < c.world) {
      uint32_t* cnt = rs_counter(c, c.rank, parity, threadIdx.x, t);
      bool got = false;
      const long long t0 = clock64();
      for (long long i = 0; !got; ++i) {
        got = ld_acquire_sys(cnt) >= static_cast<uint32_t>(n_tiles);
        if (!got) {
          if (i > (1 << 14)) __nanosleep(64);
          if ((i & 255) == 255 && clock64() - t0 > 4000000000ll) break;
        }
      }
      if (!got) {
        if (atomicCAS(&status->code, 0, kTimeoutPeerFlag) == 0) status->detail = 200 + threadIdx.x;
        atomicAdd(&status->count, 1);
        ok_s = 0;
      }
    }
    __syncthreads();
    if (ok_s) {
      // four independent 16-byte vectors per thread and iteration: the loop is bound by memory latency, not by math
      constexpr int U = 4;
      const int items = rows * vec;
      for (int i0 = threadIdx.x; i0 < items; i0 += blockDim.x * U) {
        size_t off[U];
        float acc[U][8];
        Pack16 xr[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = min(i0 + u * static_cast<int>(blockDim.x), items - 1);      // clamped: tail lanes repeat an item
          off[u] = (static_cast<size_t>(r0 + i / vec) * H + c0) * 2 + static_cast<size_t>(i % vec) * 16;
          xr[u].u = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(x) + off[u]);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
        }
        for (int s = 0; s < c.world; ++s) {
          Pack16 pk[U];
          // L2 is the coherence point of the peers' stores: .cg loads skip L1 and, unlike volatile ones, pipeline
#pragma unroll
          for (int u = 0; u < U; ++u) pk[u].u = __ldcg(reinterpret_cast<const uint4*>(payload(c, c.rank, parity, s) + off[u]));
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[u][j] += bf16_to_f32(pk[u].h[j]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (i0 + u * static_cast<int>(blockDim.x) >= items) break;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            xr[u].h[j] = f32_to_bf16(bf16_to_f32(xr[u].h[j]) + bf16_to_f32(f32_to_bf16(acc[u][j])));
          *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(x) + off[u]) = xr[u].u;
          for (int d = 1; d < c.world; ++d) {
            const int dst = (c.rank + d) % c.world;
            st_v4_global(payload(c, dst, parity, c.rank) + off[u], xr[u].u);
          }
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < c.world && threadIdx.x != c.rank && ok_s)
      st_release_sys(ag_flag(c, threadIdx.x, parity, t, chunk), epoch);
    // the last column chunk of this tile zeroes the arrival counters for the next use of this parity
    if (threadIdx.x == 0) {
      if (atomicAdd(rs_local_done(c, t), 1u) == static_cast<uint32_t>(chunks - 1)) {
        *rs_local_done(c, t) = 0;
        for (int s = 0; s < c.world; ++s) *rs_counter(c, c.rank, parity, s, t) = 0;
        __threadfence_system();
      }
    }
  } else {
    if (threadIdx.x == 0 && !wait_flag(ag_flag(c, c.rank, parity, t, chunk), epoch)) {
      if (atomicCAS(&status->code, 0, kTimeoutPeerFlag) == 0) status->detail = 300 + owner;
      atomicAdd(&status->count, 1);
      ok_s = 0;
    }
    __syncthreads();
    if (ok_s) {
      constexpr int U = 4;
      const int items = rows * vec;
      for (int i0 = threadIdx.x; i0 < items; i0 += blockDim.x * U) {
        size_t off[U];
        uint4 val[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int i = min(i0 + u * static_cast<int>(blockDim.x), items - 1);
          off[u] = (static_cast<size_t>(r0 + i / vec) * H + c0) * 2 + static_cast<size_t>(i % vec) * 16;
          val[u] = __ldcg(reinterpret_cast<const uint4*>(payload(c, c.rank, parity, owner) + off[u]));
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * static_cast<int>(blockDim.x) < items)
            *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(x) + off[u]) = val[u];
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(c.done_ctas, 1u) == gridDim.x * gridDim.y - 1) {
      *c.done_ctas = 0;
      *c.epoch = epoch;
      __threadfence();
    }
  }
}

// Sequence-parallel boundary: reduce-scatter fold + residual add + RMSNorm at the owner, all-gather of the NORMED rows.
// One CTA per row of this rank's OWN token tiles (the residual stream stays sharded by token tile: a rank only ever
// needs the residual of the rows it folds).  The CTA waits (bounded) until every rank has delivered all `n_tiles` output
// tiles of the row's token tile, folds the W partial rows in ascending rank order (fp32, one bf16 rounding), adds the
// residual, stores the new residual row locally, normalises it with the arithmetic of rmsnorm_kernel (same thread ->
// element map and reduction tree, so the fused and the separate path agree bit for bit) and stores the normed row into
// slot `rank` of EVERY rank's region (its own included) at the row's offset: rows of a source slot that the
// reduce-scatter does not use.  The last CTA of a token tile raises the peers' all-gather flag of that tile; the consumer
// GEMM (gemm_tc all-gather mode) waits for the flag in its TMA producer warp and reads the rows where they landed, so
// there is no copy pass and local tiles start at once.
__global__ void __launch_bounds__(256)
rs_norm_push_kernel(CommState c, bf16* __restrict__ x, const bf16* __restrict__ w, float eps, int one_plus_w, int T, int H,
                    int tile_rows, int tiles_per_rank, int n_tiles, int row_begin, DeviceStatus* status) {
  extern __shared__ __align__(16) unsigned char rs_smem[];
  bf16* row_s = reinterpret_cast<bf16*>(rs_smem);
  __shared__ float scratch[32];
  __shared__ int ok_s;
  pdl_wait();
  const uint32_t epoch = *c.epoch + 1;
  const int parity = epoch & 1;
  const int row = row_begin + blockIdx.x;
  const int t = row / tile_rows;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    uint32_t* cnt = rs_counter(c, c.rank, parity, threadIdx.x, t);
    bool got = false;
    const long long t0 = clock64();
    for (long long i = 0; !got; ++i) {
      got = ld_acquire_sys(cnt) >= static_cast<uint32_t>(n_tiles);
      if (!got) {
        if (i > (1 << 14)) __nanosleep(64);
        if ((i & 255) == 255 && clock64() - t0 > 4000000000ll) break;
      }
    }
    if (!got) {
      if (atomicCAS(&status->code, 0, kTimeoutPeerFlag) == 0) status->detail = 400 + threadIdx.x;
      atomicAdd(&status->count, 1);
      ok_s = 0;
    }
  }
  __syncthreads();
  const int nvec = H / 8;
  const size_t off = static_cast<size_t>(row) * H * 2;
  float ss = 0.f;
  if (ok_s) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int s = 0; s < c.world; ++s) {
        Pack16 pk;
        pk.u = __ldcg(reinterpret_cast<const uint4*>(payload(c, c.rank, parity, s) + off) + i);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += bf16_to_f32(pk.h[j]);
      }
      Pack16 a;
      a.u = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(x) + off)[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a.h[j] = f32_to_bf16(bf16_to_f32(a.h[j]) + bf16_to_f32(f32_to_bf16(acc[j])));
        const float f = bf16_to_f32(a.h[j]);
        ss += f * f;
      }
      reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(x) + off)[i] = a.u;
      reinterpret_cast<uint4*>(row_s)[i] = a.u;
    }
  }
  // block sum in the order of rmsnorm_kernel: lanes by xor tree, then warps ascending
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) total += scratch[i];
  const float rstd = rsqrtf(total / static_cast<float>(H) + eps);
  if (ok_s) {
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      Pack16 a, ww, o;
      a.u = reinterpret_cast<const uint4*>(row_s)[i];
      ww.u = reinterpret_cast<const uint4*>(w)[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float n = bf16_to_f32(f32_to_bf16(bf16_to_f32(a.h[j]) * rstd));
        float g = bf16_to_f32(ww.h[j]);
        if (one_plus_w) g += 1.f;
        o.h[j] = f32_to_bf16(n * g);
      }
      for (int d = 0; d < c.world; ++d) {
        const int dst = (c.rank + d) % c.world;
        st_v4_global(payload(c, dst, parity, c.rank) + off + static_cast<size_t>(i) * 16, o.u);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int rows_in_tile = min(tile_rows, T - t * tile_rows);
    if (atomicAdd(rs_local_done(c, t), 1u) == static_cast<uint32_t>(rows_in_tile - 1)) {
      *rs_local_done(c, t) = 0;
      for (int s = 0; s < c.world; ++s) *rs_counter(c, c.rank, parity, s, t) = 0;
      __threadfence_system();
      if (ok_s)
        for (int d = 1; d < c.world; ++d) st_release_sys(ag_flag(c, (c.rank + d) % c.world, parity, t, 0), epoch);
    }
    __threadfence();
    if (atomicAdd(c.done_ctas, 1u) == gridDim.x - 1) {
      *c.done_ctas = 0;
      *c.epoch = epoch;
      __threadfence();
    }
  }
}

// A rank that owns no row of this exchange still has to close the epoch.
__global__ void rs_epoch_only_kernel(CommState c) {
  pdl_wait();
  if (threadIdx.x == 0) {
    *c.epoch = *c.epoch + 1;
    __threadfence();
  }
}

}  // namespace dgpp

using namespace dgpp;


static size_t region_size(int world, size_t slot_bytes) {
  const size_t rs_tables = (2 * static_cast<size_t>(world) * kCommMaxCtas + 2 * static_cast<size_t>(kCommMaxCtas) * kRsMaxChunks +
                            kCommMaxCtas) * sizeof(uint32_t);
  return 2 * static_cast<size_t>(world) * slot_bytes + 2 * static_cast<size_t>(world) * kCommMaxCtas * sizeof(uint32_t) +
         2 * static_cast<size_t>(world) * kPickRows * 8 + 2 * static_cast<size_t>(world) * sizeof(uint32_t) + 512 + rs_tables;
}

// Step 1: allocate the local symmetric region; returns the comm handle and writes the 64-byte IPC handle.
DGPP_API void* dgpp_comm_create(int world, int rank, int64_t slot_bytes, void* ipc_handle_out) {
  if (world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world || slot_bytes % 16 != 0) {
    dgpp_set_error("comm_create: bad arguments (world %d rank %d slot %lld)", world, rank, (long long)slot_bytes);
    return nullptr;
  }
  DgppComm* c = new DgppComm();
  memset(c, 0, sizeof(*c));
  c->region_bytes = region_size(world, static_cast<size_t>(slot_bytes));
  if (cudaMalloc(&c->local, c->region_bytes) != cudaSuccess || cudaMemset(c->local, 0, c->region_bytes) != cudaSuccess) {
    dgpp_set_error("comm_create: cudaMalloc of %zu bytes failed", c->region_bytes);
    delete c;
    return nullptr;
  }
  uint32_t* counters = nullptr;
  if (cudaMalloc(&counters, 64) != cudaSuccess || cudaMemset(counters, 0, 64) != cudaSuccess) {
    dgpp_set_error("comm_create: counter allocation failed");
    cudaFree(c->local);
    delete c;
    return nullptr;
  }
  c->st.world = world;
  c->st.rank = rank;
  c->st.slot_bytes = static_cast<size_t>(slot_bytes);
  c->st.epoch = counters;
  c->st.done_ctas = counters + 1;
  c->st.pick_epoch = counters + 2;
  c->st.peers[rank] = static_cast<unsigned char*>(c->local);
  if (world > 1) {
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, c->local) != cudaSuccess) {
      dgpp_set_error("comm_create: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(cudaGetLastError()));
      cudaFree(c->local);
      cudaFree(counters);
      delete c;
      return nullptr;
    }
    memcpy(ipc_handle_out, &h, sizeof(h));
  }
  cudaDeviceSynchronize();
  return c;
}

// Step 2: map the regions of all peers.  handles: world x 64 bytes, in rank order.
DGPP_API int dgpp_comm_connect(void* comm, const void* handles) {
  DgppComm* c = static_cast<DgppComm*>(comm);
  for (int r = 0; r < c->st.world; ++r) {
    if (r == c->st.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const unsigned char*>(handles) + r * sizeof(h), sizeof(h));
    void* p = nullptr;
    DGPP_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->opened[r] = p;
    c->st.peers[r] = static_cast<unsigned char*>(p);
  }
  return 0;
}

// Single-GPU stand-in for the peers: every rank slot that has no mapping yet points at this rank's own region.
// Pushes then land in the local region and the flags of the other source ranks are never raised, which is how the
// bounded-wait / status path is exercised without a second process (a missing peer looks exactly like this).
DGPP_API int dgpp_comm_loopback(void* comm) {
  DgppComm* c = static_cast<DgppComm*>(comm);
  for (int r = 0; r < c->st.world; ++r)
    if (!c->st.peers[r]) c->st.peers[r] = static_cast<unsigned char*>(c->local);
  return 0;
}

DGPP_API int dgpp_comm_destroy(void* comm) {
  DgppComm* c = static_cast<DgppComm*>(comm);
  if (!c) return 0;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->st.world; ++r)
    if (c->opened[r]) cudaIpcCloseMemHandle(c->opened[r]);
  cudaFree(c->st.epoch);
  cudaFree(c->local);
  delete c;
  return 0;
}

// In-place sum of `n` bf16 values over all ranks (n * 2 <= slot_bytes, n % 8 == 0); optional fused residual.
DGPP_API int dgpp_comm_all_reduce(void* comm, void* data, const void* resid, int64_t n, int ctas, cudaStream_t st) {
  DgppComm* c = static_cast<DgppComm*>(comm);
  DGPP_REQUIRE(n % 8 == 0, "all_reduce: n %lld must be a multiple of 8", (long long)n);
  DGPP_REQUIRE(static_cast<size_t>(n) * 2 <= c->st.slot_bytes, "all_reduce: %lld values exceed the slot", (long long)n);
  if (ctas < 1) ctas = 1;
  if (ctas > kCommMaxCtas) ctas = kCommMaxCtas;
  ar_oneshot_kernel<<<ctas, 256, 0, st>>>(c->st, static_cast<bf16*>(data), static_cast<const bf16*>(resid), n,
                                         device_status_ptr());
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Geometry of the reduce-scatter: token tiles of `tile_rows` rows are dealt to ranks in runs of tiles_per_rank.
static int rs_tiles_per_rank(int T, int tile_rows, int world) {
  const int tiles = dgpp_ceil_div(T, tile_rows);
  return dgpp_ceil_div(tiles, world);
}

// x [T, H] += sum over ranks of the partial tiles the preceding dgpp_gemm_tc(..., comm_push) calls delivered.
DGPP_API int dgpp_comm_rs_ag(void* comm, void* x, int T, int H, int tile_rows, cudaStream_t st) {
  DgppComm* c = static_cast<DgppComm*>(comm);
  const int tiles = dgpp_ceil_div(T, tile_rows);
  DGPP_REQUIRE(T > 0 && tiles <= kCommMaxCtas, "rs_ag: %d rows in tiles of %d exceed %d token tiles", T, tile_rows, kCommMaxCtas);
  DGPP_REQUIRE(H % 128 == 0, "rs_ag: hidden %d must be a multiple of 128", H);
  DGPP_REQUIRE(static_cast<size_t>(T) * H * 2 <= c->st.slot_bytes, "rs_ag: %d x %d exceeds the slot", T, H);
  int chunks = 1;
  for (int cand : {16, 8, 5, 4, 2})
    if (cand <= kRsMaxChunks && H % (cand * 8) == 0 && tiles * cand <= 592) { chunks = cand; break; }
  rs_ag_kernel<<<dim3(tiles, chunks), 256, 0, st>>>(c->st, static_cast<bf16*>(x), T, H, tile_rows,
                                                    rs_tiles_per_rank(T, tile_rows, c->st.world), H / 128,
                                                    device_status_ptr());
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Sequence-parallel form of the boundary (see rs_norm_push_kernel): x [T, H] keeps only this rank's token tiles up to
// date; the normed rows of ALL tiles land in every rank's region, where dgpp_gemm_tc_ag reads them.
DGPP_API int dgpp_comm_rs_norm_push(void* comm, void* x, const void* norm_w, float eps, int one_plus_w, int T, int H,
                                    int tile_rows, cudaStream_t st) {
  DgppComm* c = static_cast<DgppComm*>(comm);
  const int tiles = dgpp_ceil_div(T, tile_rows);
  DGPP_REQUIRE(T > 0 && tiles <= kCommMaxCtas, "rs_norm_push: %d rows in tiles of %d exceed %d token tiles", T, tile_rows, kCommMaxCtas);
  DGPP_REQUIRE(H % 128 == 0 && H * 2 <= 96 * 1024, "rs_norm_push: hidden %d must be a multiple of 128 (<= 48K)", H);
  DGPP_REQUIRE(static_cast<size_t>(T) * H * 2 <= c->st.slot_bytes, "rs_norm_push: %d x %d exceeds the slot", T, H);
  const int tpr = rs_tiles_per_rank(T, tile_rows, c->st.world);
  const int own0 = c->st.rank * tpr < tiles ? c->st.rank * tpr : tiles;
  const int own1 = c->st.rank == c->st.world - 1 ? tiles : ((c->st.rank + 1) * tpr < tiles ? (c->st.rank + 1) * tpr : tiles);
  const int r0 = own0 * tile_rows;
  const int r1 = own1 * tile_rows < T ? own1 * tile_rows : T;
  if (r1 <= r0) {
    rs_epoch_only_kernel<<<1, 32, 0, st>>>(c->st);
    DGPP_CUDA_OK(cudaGetLastError());
    return 0;
  }
  static bool attr = false;
  if (!attr) {
    DGPP_CUDA_OK(cudaFuncSetAttribute(rs_norm_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    attr = true;
  }
  rs_norm_push_kernel<<<r1 - r0, 256, static_cast<size_t>(H) * 2, st>>>(c->st, static_cast<bf16*>(x), static_cast<const bf16*>(norm_w),
                                                                      eps, one_plus_w, T, H, tile_rows, tpr, H / 128, r0,
                                                                      device_status_ptr());
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_comm_pick_merge(void* comm, void* ids, void* vals, int rows, cudaStream_t st) {
  DgppComm* c = static_cast<DgppComm*>(comm);
  DGPP_REQUIRE(rows >= 1 && rows <= kPickRows, "pick_merge: rows %d outside 1..%d", rows, kPickRows);
  pick_merge_kernel<<<1, 256, 0, st>>>(c->st, static_cast<int32_t*>(ids), static_cast<float*>(vals), rows,
                                      device_status_ptr());
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
