// Speculative decoding transaction on the device: greedy verdict and state commit.
//
//   spec_accept_kernel   rows come in runs of V per request: row 0 carries the pending (already emitted) token, rows
//                        1..V-1 the drafts.  picks[r, i] is the model's greedy token after row i.  A draft is accepted while
//                        it equals the pick of the row before it; n_acc[r] = 1 + accepted drafts (rows whose state is kept),
//                        emitted[r, 0..n_acc) = the picks of the kept rows (the new tokens of this step), -1 beyond.
//   spec_commit_kernel   recurrent layers advanced their state through all V rows and saved it after every row; for a run
//                        with n_acc < V the live state of its slot is replaced by the snapshot after row n_acc - 1
//                        (conditional rollback copy; a fully accepted run is left alone).  One launch covers every
//                        recurrent layer (pooled state and snapshot tensors).
// The paged KV rows of rejected drafts need no undo: they sit beyond the committed length and are overwritten.
// (reference counterparts: src/kernels/glm_spec.cu:48 spec_commit_kernel, src/engine/speculative.hpp greedy verdict.)
#include "common/common.h"
#include "common/ptx.cuh"

namespace dgpp {

__global__ void spec_accept_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ picks,
                                   int32_t* __restrict__ n_acc, int32_t* __restrict__ emitted, int R, int V) {
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  int n = 1;
  while (n < V && tokens[r * V + n] == picks[r * V + n - 1]) ++n;
  n_acc[r] = n;
  for (int i = 0; i < V; ++i) emitted[r * V + i] = i < n ? picks[r * V + i] : -1;
}

// grid (ceil(max(S, C) / 4 / 256), R, layers).  state: [layers, slots, S] fp32, snap: [layers, rows, S]; same for the
// convolution tails with C values.  S and C are multiples of 4.
__global__ void __launch_bounds__(256) spec_commit_kernel(float* __restrict__ ssm, const float* __restrict__ ssm_snap,
                                                          float* __restrict__ conv, const float* __restrict__ conv_snap,
                                                          const int32_t* __restrict__ run_slot, const int32_t* __restrict__ n_acc,
                                                          int slots, int rows, int V, int64_t S, int64_t C) {
  pdl_wait();
  const int r = blockIdx.y, l = blockIdx.z;
  const int n = n_acc[r];
  if (n >= V) return;
  const int slot = run_slot[r * V];
  const int64_t row = static_cast<int64_t>(r) * V + n - 1;
  const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (v * 4 < S) {
    const float4 x = reinterpret_cast<const float4*>(ssm_snap + (static_cast<int64_t>(l) * rows + row) * S)[v];
    reinterpret_cast<float4*>(ssm + (static_cast<int64_t>(l) * slots + slot) * S)[v] = x;
  }
  if (v * 4 < C) {
    const float4 x = reinterpret_cast<const float4*>(conv_snap + (static_cast<int64_t>(l) * rows + row) * C)[v];
    reinterpret_cast<float4*>(conv + (static_cast<int64_t>(l) * slots + slot) * C)[v] = x;
  }
}

}  // namespace dgpp

using namespace dgpp;

DGPP_API int dgpp_spec_accept(const void* tokens, const void* picks, void* n_acc, void* emitted, int R, int V, cudaStream_t st) {
  DGPP_REQUIRE(R >= 1 && V >= 1, "spec_accept: bad sizes %d x %d", R, V);
  spec_accept_kernel<<<dgpp_ceil_div(R, 64), 64, 0, st>>>(static_cast<const int32_t*>(tokens), static_cast<const int32_t*>(picks),
                                                          static_cast<int32_t*>(n_acc), static_cast<int32_t*>(emitted), R, V);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}

DGPP_API int dgpp_spec_commit(void* ssm, const void* ssm_snap, void* conv, const void* conv_snap, const void* run_slot,
                              const void* n_acc, int layers, int slots, int rows, int R, int V, int64_t S, int64_t C,
                              cudaStream_t st) {
  DGPP_REQUIRE(S % 4 == 0 && C % 4 == 0 && R * V <= rows && layers >= 1, "spec_commit: bad sizes");
  const int64_t m = (S > C ? S : C) / 4;
  dim3 grid(static_cast<unsigned>(dgpp_ceil_div64(m, 256)), R, layers);
  spec_commit_kernel<<<grid, 256, 0, st>>>(static_cast<float*>(ssm), static_cast<const float*>(ssm_snap),
                                           static_cast<float*>(conv), static_cast<const float*>(conv_snap),
                                           static_cast<const int32_t*>(run_slot), static_cast<const int32_t*>(n_acc), slots, rows,
                                           V, S, C);
  DGPP_CUDA_OK(cudaGetLastError());
  return 0;
}
