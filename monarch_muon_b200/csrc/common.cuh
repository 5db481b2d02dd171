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

// Largest grid of the streaming (bandwidth-bound) kernels: 32 CTAs of 256 threads per SM by default,
// fewer after mmb_set_stream_ctas_per_sm(n) - used when they run beside the persistent GEMMs, whose
// CTAs leave room for one small CTA per SM.
void set_stream_ctas_per_sm(int n);
long long stream_grid_cap(int sms);

// True while mmb_set_stream_ctas_per_sm() is in force: streaming kernels then ask for the same shared
// memory carve-out as the persistent GEMMs (the maximum), because an SM cannot hold kernels of two
// different carve-outs at once and would otherwise drain the GEMM CTA before admitting them.
bool stream_kernels_share_sms();

// Tile schedule of the Newton-Schulz GEMMs: static round-robin (default) or drawn from a counter
// (mmb_set_gemm_schedule).
void set_gemm_schedule_dynamic(bool on);
bool gemm_schedule_dynamic();

// Newton-Schulz GEMMs are launched with programmatic stream serialisation (default) or plainly
// (mmb_set_gemm_dependent_launch).
void set_gemm_dependent_launch(bool on);
bool gemm_dependent_launch();

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
  STATUS_WAIT_PROBE = 0x1F0,           // mmb_wait_probe(): the deliberately unanswered wait expired, as it must
};

#ifdef __CUDACC__
// Threads per CTA of a bandwidth-bound kernel.  While mmb_set_stream_ctas_per_sm() is in force they are meant
// to sit on an SM beside a Newton-Schulz GEMM CTA (13 warps of 112 registers and nearly all shared memory).
// What that leaves per SM sub-partition is 2048 registers on the one that holds four GEMM warps, so a guest
// CTA fits if it puts one warp of at most 64 registers on each sub-partition: 128 threads.  Kernels launched
// through launch_stream_kernel index by blockDim, not by a constant.
inline int stream_threads(int normal) { return stream_kernels_share_sms() ? 128 : normal; }

// Launch of a bandwidth-bound kernel (no dynamic shared memory) with the carve-out and CTA size that fit the
// mode; `grid` must have been sized for stream_threads(threads) threads per CTA.
template <typename... KArgs, typename... Args>
inline void launch_stream_kernel(void (*kernel)(KArgs...), int grid, int threads, cudaStream_t st, Args... args) {
  cudaFuncSetAttribute(reinterpret_cast<const void*>(kernel), cudaFuncAttributePreferredSharedMemoryCarveout,
                       stream_kernels_share_sms() ? static_cast<int>(cudaSharedmemCarveoutMaxShared)
                                                  : static_cast<int>(cudaSharedmemCarveoutDefault));
  kernel<<<grid, stream_threads(threads), 0, st>>>(args...);
}
#endif

}  // namespace mmb
