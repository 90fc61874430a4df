// C ABI of the persistent decode-layer kernel (decode_layer.cu): a launch walks a list of phases over one grid
// of (number of SMs) CTAs; see the kernel file for what each phase does.
#pragma once
#include <stdint.h>

#include "common/common.h"

enum {
  kDlPhRowA = 1,    // one CTA per (row, column segment): produce the slice of an activation row + partial row statistics
  kDlPhGemm = 2,    // block-scaled NVFP4 GEMM over (weight tile, K split) work items
  kDlPhUnitq = 3,   // quantise the SwiGLU output written by a gate/up GEMM phase
  kDlPhRope = 4,    // per-head RMSNorm + RoPE + KV append of a qkv GEMM phase
  kDlPhRowC = 5,    // finishing step of the preceding kDlPhRowA phase: row statistics -> RMSNorm, quantise the slice
};
enum { kDlMaxPhase = 16, kDlMaxGemm = 4, kDlMaxAct = 3, kDlMaxRowq = 3 };

// Quantised activation buffer: 16 token rows x 3 residual terms (rows of `q` ordered [term][token], K / 2 bytes each),
// block scales in tcgen05.cp atom order, one fp32 row scale per token.  Rows that are never written must be zero.
struct DgppDlAct {
  void* q;
  void* sf;
  void* g;
  int K;
  int pad;
};
// Weight matrix [N, K] as packed e2m1, STAGE-TILED: [N / 128][K / 256][128 rows][128 bytes] (each 128-row x 256-K
// stage contiguous), with tiled e4m3 block scales; `act` names the activation buffer it multiplies.
// pair = 1: rows [0, N/2) are the gate and [N/2, N) the up projection; the phase writes bf16 SwiGLU rows + row maxima.
// splits = 0: chosen so that (tiles x splits) fills the grid.
struct DgppDlGemm {
  const void* wq;
  const void* wsf;
  float alpha;
  int N, K, pair, act, splits;
};
// mode 0: rows of `in` (bf16);  mode 2: x += fold(src_gemm partials [, across ranks]); rmsnorm(x) * norm_w;
// mode 3: fold of the split-KV attention partials.  The row is quantised into activation `out_act` (-1: not) and,
// when x_out is given, also stored there as bf16.
struct DgppDlRowq {
  int mode, src_gemm, out_act, tp_fold;
  const void* in;
  int64_t in_stride;
  const void* norm_w;
  void* x_out;
};
struct DgppDecodeLayerArgs {
  int rows, nphase;
  int ph_type[kDlMaxPhase];
  int ph_idx[kDlMaxPhase];
  DgppDlGemm gemm[kDlMaxGemm];
  DgppDlAct act[kDlMaxAct];
  DgppDlRowq rowq[kDlMaxRowq];
  void* x;                 // residual stream [rows, H] bf16, updated in place by mode-2 row phases
  int H;
  float eps, limit;
  int one_plus_w;
  void* ws;                // fp32 split-K partials [splits][16][N]
  int64_t ws_floats;
  void* hbuf;              // bf16 SwiGLU rows [rows, inter]
  void* amax_part;         // fp32 [inter / 128][16]
  void* stats;             // fp32 [16][8][2] scratch of the row phases
  int unitq_act, inter;
  const void* part_ml;     // split-KV attention partials (mode 3)
  const void* part_acc;
  int att_splits, hq, d;
  int rope_gemm, hkv;
  void* qkv;               // bf16 [rows, (hq + 2 hkv) * d]: rotated q / k and v of the RoPE phase
  const void* positions;
  const void* row_req;
  const void* block_table;
  const void* inv_freq;
  const void* q_norm_w;
  const void* k_norm_w;
  void* k_cache;
  void* v_cache;
  void* k_scale;
  void* v_scale;
  int rot_dim, page, max_blocks, kv_fp8;
  float mscale;
  int grid;                // 0: one CTA per SM
  void* comm;              // DgppComm* of the tensor-parallel group, or null
};

DGPP_API int dgpp_decode_layer(const DgppDecodeLayerArgs* a, cudaStream_t st);
DGPP_API int dgpp_decode_layer_reset(cudaStream_t st);
DGPP_API int dgpp_decode_layer_grid();
DGPP_API int dgpp_decode_layer_set_trace(void* dev_u64x64);
