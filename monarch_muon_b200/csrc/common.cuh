// Shared host/device helpers for libmonarch_muon_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/monarch_muon_b200.h"

namespace mmb {

// Thread-local message behind mmb_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define MMB_CUDA_CHECK(expr)                                                                  \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return ::mmb::fail(MMB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                         __FILE__, __LINE__);                                                 \
  } while (0)

#define MMB_REQUIRE(cond, ...)                                   \
  do {                                                           \
    if (!(cond)) return ::mmb::fail(MMB_ERR_INVALID, __VA_ARGS__); \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs kernels may size their grids for: the device's count, or the limit set with
// mmb_set_sm_limit() if that is smaller.
int sm_count();
void set_sm_limit(int n);

// Tile schedule of the Newton-Schulz GEMMs: static round-robin (default) or drawn from a counter
// (mmb_set_gemm_schedule).
void set_gemm_schedule_dynamic(bool on);
bool gemm_schedule_dynamic();

// Device scalar that the momentum and AdamW kernels multiply gradients by (mmb_set_device_grad_scale),
// or null.  Thread local, like the error message.
const float* device_grad_scale();
void set_device_grad_scale(const float* p);

// Process-wide count of kernels this library has launched (mmb_launch_count()).
void count_launch(int n = 1);

// Device status codes stored by kernels (first writer wins).
enum : int32_t {
  STATUS_OK = 0,
  STATUS_WAIT_PRODUCER_EMPTY = 0x101,  // TMA producer waited too long for a free stage
  STATUS_WAIT_MMA_FULL = 0x102,        // MMA issuer waited too long for operands
  STATUS_WAIT_MMA_TMEM_EMPTY = 0x103,  // MMA issuer waited too long for a drained accumulator
  STATUS_WAIT_EPI_TMEM_FULL = 0x104,   // epilogue waited too long for an accumulator
  STATUS_WAIT_SCHED_FULL = 0x105,      // a role waited too long for its next tile number
  STATUS_WAIT_SCHED_EMPTY = 0x106,     // the tile scheduler waited too long for a slot to be returned
};

}  // namespace mmb
