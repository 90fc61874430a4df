// Split-KV paged decode attention with the split scratch in a fixed device array: an entry point that allocates
// nothing.  This entry point has NO counterpart in the reference engine (whose attention launchers take their
// scratch from an arena owned by the caller); it exists for hosts that must call the kernel from a context where
// no allocator may run (no cudaMalloc / cudaFree, no framework tensor).
//
// Contract
//   * Same arguments and the same result, bit for bit, as dgpp_attn_decode(), minus the two scratch pointers.
//   * The scratch is one file-scope `static __device__` array of kAttnStaticScratchFloats floats (4 MiB) per
//     device context.  A call needs rows * hq * splits * 2 floats for the (max, sum) pairs, rounded up to a
//     multiple of 64 floats, plus rows * hq * splits * head_dim floats for the partial outputs; a call that needs
//     more is rejected with a non-zero return and a message (dgpp_last_error) that states both numbers.  Nothing
//     is launched in that case.
//   * Set-up: the first call on each device resolves the array's address with cudaGetSymbolAddress (which also
//     loads the module on that device).  Make that first call BEFORE any stream capture begins; later calls on the
//     same device only launch kernels.
//   * The array is shared by every call on the device and keeps whatever the last call left in it.  The kernels
//     write every scratch element they later read, so nothing in it has to start at zero and no call clears it.
//   * Two calls that overlap in time on one device (different streams, or different host threads) race on the
//     array: serialise them on one stream or order them with events.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Number of floats in the fixed scratch array (per device).
#define DGPP_ATTN_STATIC_SCRATCH_FLOATS (1u << 20)

__attribute__((visibility("default")))
int dgpp_attn_decode_static(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                            const void* k_scale, const void* v_scale, const void* block_table, const void* row_req,
                            const void* positions, void* out, int rows, int hq, int hkv, int d, int page,
                            int max_blocks, int splits, int kv_fp8, float scale, int window, cudaStream_t st);

#ifdef __cplusplus
}
#endif
