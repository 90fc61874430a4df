// Expert parallelism with an all-to-all over NVLink peer memory: tokens are sharded over the ranks (every rank routes
// ITS rows), experts are sharded over the ranks (rank r owns experts [r E / W, (r + 1) E / W)).
//
//   source                                              owner of the expert
//   ------                                              -------------------
//   ep_plan_kernel       (token, k) pairs -> destination rank, position in that rank's receive list (stable)
//   ep_dispatch_kernel   pair rows + (local expert, pair index) stored into the owner's receive area  ----->
//                        last CTA: row counts, then the "dispatched" flag on every owner
//                                                       ep_recv_plan_kernel   bounded wait for W flags; received ids in
//                                                                             (source, position) order
//                                                       [segment sort into tiles, ep_gather_kernel, quantise, grouped
//                                                        block-scaled GEMMs: the single-rank prefill path's kernels]
//                              <-----                   ep_return_kernel      result rows stored into the source's return
//                                                                             area at their pair index; last CTA: flags
//   ep_combine_kernel    bounded wait for W "returned" flags; out[t] = sum_j w[t, j] * row(t, j) (+ shared[t]) in
//                        ascending j, fp32, one rounding; last CTA advances the epoch
//
// Areas live in the communicator's symmetric region: slot (parity, source) of every rank is split into a receive half
// (header: count; meta table; rows) and a return half (rows by pair index).  Only plain vector stores, volatile loads
// and system-scope flags touch peer memory; every wait is bounded and reports into the status block.
// The result does not depend on arrival order: positions, tiles and the fold order are functions of the routing result.
// (reference counterparts: src/kernels/glm_moe.cu dispatch / combine kernels, src/engine/tp_bus.hpp expert exchange.)
#include "common/common.h"
#include "common/dtypes.cuh"
#include "common/ptx.cuh"
#include "kernels/comm.cuh"

namespace dgpp {

constexpr int kEpFlagDispatched = 0;
constexpr int kEpFlagReturned = 1;
constexpr int kEpPlanThreads = 1024;

struct EpGeom {
  int T, k, H, E, max_pairs;        // local rows, top-k, hidden, global experts, pair capacity of one (source, owner) area
  size_t meta_off, rows_off, ret_off;   // byte offsets inside a slot
};

__host__ __device__ inline EpGeom ep_geom(int T, int k, int H, int E, int max_pairs) {
  EpGeom g;
  g.T = T; g.k = k; g.H = H; g.E = E; g.max_pairs = max_pairs;
  g.meta_off = 256;
  g.rows_off = (g.meta_off + static_cast<size_t>(max_pairs) * 8 + 255) & ~static_cast<size_t>(255);
  g.ret_off = g.rows_off + static_cast<size_t>(max_pairs) * H * 2;
  return g;
}
__host__ __device__ inline size_t ep_slot_bytes(int H, int max_pairs) {
  const EpGeom g = ep_geom(0, 1, H, 1, max_pairs);
  return (g.ret_off + static_cast<size_t>(max_pairs) * H * 2 + 255) & ~static_cast<size_t>(255);
}
__device__ __forceinline__ int ep_owner(int e, int E, int W) { return e / (E / W); }

// One CTA.  dest_pos[p] = position of pair p among the pairs that go to the same rank (pairs keep their (t, k) order);
// dest_cnt[r] = pairs for rank r.
__global__ void __launch_bounds__(kEpPlanThreads) ep_plan_kernel(const int32_t* __restrict__ ids, int P, int E, int W,
                                                                 int32_t* __restrict__ dest_pos, int32_t* __restrict__ dest_cnt) {
  __shared__ int hist[kEpPlanThreads / 32][kCommMaxWorld];
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int kWarps = kEpPlanThreads / 32;
  const int seg = (P + kWarps - 1) / kWarps;
  const int p0 = warp * seg, p1 = min(P, p0 + seg);
  if (lane < kCommMaxWorld) hist[warp][lane] = 0;
  __syncwarp();
  for (int p = p0 + lane; p < p1; p += 32) atomicAdd(&hist[warp][ep_owner(ids[p], E, W)], 1);
  __syncthreads();
  if (tid < W) {
    int run = 0;
    for (int w = 0; w < kWarps; ++w) {
      const int c = hist[w][tid];
      hist[w][tid] = run;
      run += c;
    }
    dest_cnt[tid] = run;
  }
  __syncthreads();
  for (int base = p0; base < p1; base += 32) {
    const int p = base + lane;
    const int o = p < p1 ? ep_owner(ids[p], E, W) : -1;
    const unsigned same = __match_any_sync(0xffffffffu, o);
    const int rank_in = __popc(same & ((1u << lane) - 1u));
    const int leader = __ffs(same) - 1;
    int start = 0;
    if (o >= 0 && lane == leader) {
      start = hist[warp][o];
      hist[warp][o] = start + __popc(same);
    }
    start = __shfl_sync(0xffffffffu, start, leader);
    if (p < p1) dest_pos[p] = start + rank_in;
    __syncwarp();
  }
}

// grid (P pairs), 128 threads.
__global__ void __launch_bounds__(128) ep_dispatch_kernel(CommState c, EpGeom g, const bf16* __restrict__ x, int64_t x_stride,
                                                          const int32_t* __restrict__ ids, const int32_t* __restrict__ dest_pos,
                                                          const int32_t* __restrict__ dest_cnt) {
  pdl_wait();
  const uint32_t epoch = *c.epoch + 1;
  const int parity = epoch & 1;
  const int p = blockIdx.x;
  const int e = ids[p];
  const int o = ep_owner(e, g.E, c.world);
  const int pos = dest_pos[p];
  if (pos < g.max_pairs) {
    unsigned char* slot = payload(c, o, parity, c.rank);
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(p / g.k) * x_stride);
    unsigned char* dst = slot + g.rows_off + static_cast<size_t>(pos) * g.H * 2;
    for (int i = threadIdx.x; i < g.H / 8; i += blockDim.x) st_v4_global(dst + static_cast<size_t>(i) * 16, src[i]);
    if (threadIdx.x == 0) {
      int32_t* meta = reinterpret_cast<int32_t*>(slot + g.meta_off) + 2 * pos;
      meta[0] = e - o * (g.E / c.world);
      meta[1] = p;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(c.done_ctas, 1u) == gridDim.x - 1) {
      *c.done_ctas = 0;
      __threadfence();
      for (int r = 0; r < c.world; ++r) {
        *reinterpret_cast<volatile int32_t*>(payload(c, r, parity, c.rank)) = min(dest_cnt[r], g.max_pairs);
        __threadfence_system();
        st_release_sys(flag(c, r, parity, c.rank, kEpFlagDispatched), epoch);
      }
    }
  }
}

// One CTA on the owner.  recv_ids[i] (local expert, -1 beyond the received pairs), recv_src[i] = source * max_pairs +
// position, in (source, position) order; n_recv[0] = total, n_recv[1 + s] = first index of source s.
__global__ void __launch_bounds__(256) ep_recv_plan_kernel(CommState c, EpGeom g, int32_t* __restrict__ recv_ids,
                                                           int32_t* __restrict__ recv_src, int32_t* __restrict__ n_recv,
                                                           DeviceStatus* status) {
  __shared__ int cnt[kCommMaxWorld + 1];
  __shared__ int ok_s;
  pdl_wait();
  const uint32_t epoch = *c.epoch + 1;
  const int parity = epoch & 1;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag(c, c.rank, parity, threadIdx.x, kEpFlagDispatched), epoch)) {
      if (atomicCAS(&status->code, 0, kTimeoutPeerFlag) == 0) status->detail = threadIdx.x;
      atomicAdd(&status->count, 1);
      ok_s = 0;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int s = 0; s < c.world; ++s) {
      cnt[s] = run;
      n_recv[1 + s] = run;
      const int n = ok_s ? *reinterpret_cast<volatile int32_t*>(payload(c, c.rank, parity, s)) : 0;
      run += min(max(n, 0), g.max_pairs);
    }
    cnt[c.world] = run;
    n_recv[0] = run;
  }
  __syncthreads();
  const int cap = c.world * g.max_pairs;
  for (int i = threadIdx.x; i < cap; i += blockDim.x) {
    int s = 0;
    while (s + 1 < c.world && i >= cnt[s + 1]) ++s;
    if (i < cnt[c.world]) {
      const int pos = i - cnt[s];
      const volatile int32_t* meta = reinterpret_cast<const volatile int32_t*>(payload(c, c.rank, parity, s) + g.meta_off) + 2 * pos;
      recv_ids[i] = meta[0];
      recv_src[i] = s * g.max_pairs + pos;
    } else {
      recv_ids[i] = -1;
      recv_src[i] = -1;
    }
  }
}

// grid (W * max_pairs), 128 threads: received row i -> its tile row.
__global__ void __launch_bounds__(128) ep_gather_kernel(CommState c, EpGeom g, const int32_t* __restrict__ recv_src,
                                                        const int32_t* __restrict__ pair_row, bf16* __restrict__ xs) {
  pdl_wait();
  const int parity = (*c.epoch + 1) & 1;
  const int i = blockIdx.x;
  const int row = pair_row[i], sp = recv_src[i];
  if (row < 0 || sp < 0) return;
  const unsigned char* src = payload(c, c.rank, parity, sp / g.max_pairs) + g.rows_off +
                             static_cast<size_t>(sp % g.max_pairs) * g.H * 2;
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * g.H);
  for (int j = threadIdx.x; j < g.H / 8; j += blockDim.x) dst[j] = ld_v4_global_volatile(src + static_cast<size_t>(j) * 16);
}

// grid (W * max_pairs), 128 threads: result row of received pair i -> the source's return area at its pair index.
__global__ void __launch_bounds__(128) ep_return_kernel(CommState c, EpGeom g, const int32_t* __restrict__ recv_src,
                                                        const int32_t* __restrict__ pair_row, const bf16* __restrict__ y) {
  pdl_wait();
  const uint32_t epoch = *c.epoch + 1;
  const int parity = epoch & 1;
  const int i = blockIdx.x;
  const int row = pair_row[i], sp = recv_src[i];
  if (row >= 0 && sp >= 0) {
    const int s = sp / g.max_pairs, pos = sp % g.max_pairs;
    const volatile int32_t* meta = reinterpret_cast<const volatile int32_t*>(payload(c, c.rank, parity, s) + g.meta_off) + 2 * pos;
    const int pidx = meta[1];
    unsigned char* dst = payload(c, s, parity, c.rank) + g.ret_off + static_cast<size_t>(pidx) * g.H * 2;
    const uint4* src = reinterpret_cast<const uint4*>(y + static_cast<size_t>(row) * g.H);
    for (int j = threadIdx.x; j < g.H / 8; j += blockDim.x) st_v4_global(dst + static_cast<size_t>(j) * 16, src[j]);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(c.done_ctas, 1u) == gridDim.x - 1) {
      *c.done_ctas = 0;
      __threadfence_system();
      for (int r = 0; r < c.world; ++r) st_release_sys(flag(c, r, parity, c.rank, kEpFlagReturned), epoch);
    }
  }
}

// grid (ceil(H / 8 / 256), T), 256 threads.
__global__ void __launch_bounds__(256) ep_combine_kernel(CommState c, EpGeom g, const int32_t* __restrict__ ids,
                                                         const float* __restrict__ w, const bf16* __restrict__ shared,
                                                         bf16* __restrict__ out, DeviceStatus* status) {
  __shared__ int ok_s;
  pdl_wait();
  const uint32_t epoch = *c.epoch + 1;
  const int parity = epoch & 1;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag(c, c.rank, parity, threadIdx.x, kEpFlagReturned), epoch)) {
      if (atomicCAS(&status->code, 0, kTimeoutPeerFlag) == 0) status->detail = 100 + threadIdx.x;
      atomicAdd(&status->count, 1);
      ok_s = 0;
    }
  }
  __syncthreads();
  const int t = blockIdx.y;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (ok_s && v * 8 < g.H) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int i = 0; i < g.k; ++i) {
      const int p = t * g.k + i;
      const int o = ep_owner(ids[p], g.E, c.world);
      const float wi = w[p];
      Pack16 r;
      r.u = ld_v4_global_volatile(payload(c, c.rank, parity, o) + g.ret_off + (static_cast<size_t>(p) * g.H + v * 8) * 2);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(wi, bf16_to_f32(r.h[j]), acc[j]);
    }
    if (shared) {
      Pack16 r;
      r.u = *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * g.H + v * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += bf16_to_f32(r.h[j]);
    }
    Pack16 o8;
#pragma unroll
    for (int j = 0; j < 8; ++j) o8.h[j] = f32_to_bf16(acc[j]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * g.H + v * 8) = o8.u;
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

}  // namespace dgpp

using namespace dgpp;

// Bytes of one (parity, source) slot for a communicator that carries `max_pairs` pairs of `H` values per exchange.
DGPP_API int64_t dgpp_ep_slot_bytes(int H, int max_pairs) { return static_cast<int64_t>(ep_slot_bytes(H, max_pairs)); }

static int ep_check(const DgppComm* c, int T, int k, int H, int E, int max_pairs) {
  DGPP_REQUIRE(c != nullptr, "ep: communicator required");
  DGPP_REQUIRE(H % 8 == 0 && E % c->st.world == 0 && k >= 1 && T >= 0 && T * k <= max_pairs,
               "ep: bad sizes (T %d k %d H %d E %d world %d capacity %d)", T, k, H, E, c->st.world, max_pairs);
  DGPP_REQUIRE(ep_slot_bytes(H, max_pairs) <= c->st.slot_bytes, "ep: %d pairs of %d values exceed the slot", max_pairs, H);
  return 0;
}

// Source side, first half: plan + dispatch of this rank's T rows.  dest_pos [T * k], dest_cnt [world] are scratch.
DGPP_API int dgpp_ep_dispatch(void* comm, const void* x, int64_t x_stride, const void* ids, void* dest_pos, void* dest_cnt,
                              int T, int k, int H, int E, int max_pairs, cudaStream_t st) {
  const DgppComm* c = static_cast<const DgppComm*>(comm);
  if (ep_check(c, T, k, H, E, max_pairs)) return -1;
  const EpGeom g = ep_geom(T, k, H, E, max_pairs);
  // a rank with no rows still raises its flags: one CTA that writes nothing
  ep_plan_kernel<<<1, kEpPlanThreads, 0, st>>>(static_cast<const int32_t*>(ids), T * k, E, c->st.world,
                                               static_cast<int32_t*>(dest_pos), static_cast<int32_t*>(dest_cnt));
  DGPP_CUDA_OK(cudaGetLastError());
  DGPP_REQUIRE(T * k >= 1, "ep_dispatch: a rank needs at least one row per exchange");
  ep_dispatch_kernel<<<T * k, 128, 0, st>>>(c->st, g, static_cast<const bf16*>(x), x_stride, static_cast<const int32_t*>(ids),
                                            static_cast<const int32_t*>(dest_pos), static_cast<const int32_t*>(dest_cnt));
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Owner side: wait for every source, list the received pairs.  recv_ids / recv_src: [world * max_pairs]; n_recv: [1 + world].
DGPP_API int dgpp_ep_recv_plan(void* comm, void* recv_ids, void* recv_src, void* n_recv, int k, int H, int E, int max_pairs,
                               cudaStream_t st) {
  const DgppComm* c = static_cast<const DgppComm*>(comm);
  if (ep_check(c, 0, k, H, E, max_pairs)) return -1;
  ep_recv_plan_kernel<<<1, 256, 0, st>>>(c->st, ep_geom(0, k, H, E, max_pairs), static_cast<int32_t*>(recv_ids),
                                         static_cast<int32_t*>(recv_src), static_cast<int32_t*>(n_recv), device_status_ptr());
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_ep_gather(void* comm, const void* recv_src, const void* pair_row, void* xs, int k, int H, int E,
                            int max_pairs, cudaStream_t st) {
  const DgppComm* c = static_cast<const DgppComm*>(comm);
  if (ep_check(c, 0, k, H, E, max_pairs)) return -1;
  ep_gather_kernel<<<c->st.world * max_pairs, 128, 0, st>>>(c->st, ep_geom(0, k, H, E, max_pairs),
                                                            static_cast<const int32_t*>(recv_src),
                                                            static_cast<const int32_t*>(pair_row), static_cast<bf16*>(xs));
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_ep_return(void* comm, const void* recv_src, const void* pair_row, const void* y, int k, int H, int E,
                            int max_pairs, cudaStream_t st) {
  const DgppComm* c = static_cast<const DgppComm*>(comm);
  if (ep_check(c, 0, k, H, E, max_pairs)) return -1;
  ep_return_kernel<<<c->st.world * max_pairs, 128, 0, st>>>(c->st, ep_geom(0, k, H, E, max_pairs),
                                                            static_cast<const int32_t*>(recv_src),
                                                            static_cast<const int32_t*>(pair_row), static_cast<const bf16*>(y));
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

// Source side, second half: wait for every owner, ordered fold into out [T, H]; advances the communicator's epoch.
DGPP_API int dgpp_ep_combine(void* comm, const void* ids, const void* w, const void* shared, void* out, int T, int k, int H,
                             int E, int max_pairs, cudaStream_t st) {
  const DgppComm* c = static_cast<const DgppComm*>(comm);
  if (ep_check(c, T, k, H, E, max_pairs)) return -1;
  DGPP_REQUIRE(T >= 1, "ep_combine: a rank needs at least one row per exchange");
  dim3 grid(dgpp_ceil_div(H / 8, 256), T);
  ep_combine_kernel<<<grid, 256, 0, st>>>(c->st, ep_geom(T, k, H, E, max_pairs), static_cast<const int32_t*>(ids),
                                          static_cast<const float*>(w), static_cast<const bf16*>(shared),
                                          static_cast<bf16*>(out), device_status_ptr());
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
