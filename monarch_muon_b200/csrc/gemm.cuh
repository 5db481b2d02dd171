// Interface between the Newton-Schulz driver and its GEMM back ends.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace mmb {

// Operand storage modes (same values as MMB_GEMM_* in the public header).
enum : int { GEMM_K = 0, GEMM_MN = 1, GEMM_SYM = 2 };

// D[b] = sigma_b * alpha * opA[b] . opB[b]^T + diag * I, bf16 in, bf16 out.
struct GemmCall {
  const void* a;
  const void* b;
  void* d;
  int batch, M, N, K;
  int a_mode, b_mode;     // GEMM_K / GEMM_MN / GEMM_SYM
  int sym_out;            // D is symmetric: only 256-blocks on or above the block diagonal are written
  float alpha, diag;
  const float* inv_norm;  // per batch, may be null
  int sigma_pow;          // sigma_b = inv_norm[b]^sigma_pow, 0..2
  int* sched = nullptr;   // two zeroed ints in device memory for the dynamic tile schedule (null: static schedule)
  // Fused Muon update (tensor-core back end): when upd_w is set the result is not written to d; block b's
  // weights upd_w[b] (M x N, row-major, 16-byte aligned) become W + upd_alpha * bf16(result) instead.
  void* const* upd_w = nullptr;
  float upd_alpha = 0.0f;
  int upd_f32 = 0;
};

int gemm_tcgen05(const GemmCall& g, int32_t* status, cudaStream_t st);
namespace tc {
// Tensor map over a bf16 array [batch][outer][inner] with a box of {64, box_outer, 1} and 128-byte swizzle.
int make_map(CUtensorMap* map, const void* base, int batch, int outer, int inner, int box_outer);
}  // namespace tc
int gemm_simt(const GemmCall& g, cudaStream_t st);
int gemm_occupancy(int pair, int* out);

// Newton-Schulz of small blocks in one launch, operands resident in shared / tensor memory (ns_onchip.cu).
bool ns_onchip_fits(int rows, int cols);
int ns_onchip(const void* x, void* out, const float* inv_norm, int batch, int rows, int cols, float beta, float kappa,
              float c, void* const* upd_w, int upd_f32, float upd_alpha, int32_t* status, cudaStream_t st);
int wait_probe(long long limit_cycles, int32_t* status, cudaStream_t st);

}  // namespace mmb
