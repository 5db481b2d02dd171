// Reduce-scatter and all-gather of the sharded optimizer step through NVSwitch multicast ("multimem").
//
// Both kernels work on a buffer that every GPU of the group has mapped at the same offset of one
// multicast object (torch.distributed's symmetric memory provides the mapping):
//
//   reduce      multimem.ld_reduce on the multicast address: the switch fetches the 16 bytes from every
//               GPU's copy, adds them as bf16 pairs with fp32 accumulation and returns one result.  A rank
//               that reads only its own shard this way performs its part of a reduce-scatter.  Per GPU the
//               links carry the whole buffer OUT once and one shard IN.
//   broadcast   multimem.st on the multicast address: the switch writes the 16 bytes into every GPU's
//               copy.  A rank that stores its own shard this way performs its part of an all-gather.  Per
//               GPU the links carry one shard OUT and the whole buffer IN.
//
// The two load opposite link directions, so a reduce of one chunk and a broadcast of another run side by
// side at full rate, which ring collectives (both directions busy in each) cannot do.  The kernels hold no
// flags and wait on nothing: ordering between ranks is the caller's (a collective on the stream before the
// first reduce of a step and after its last broadcast).
//
// Small CTAs on purpose.  The kernels run beside the Newton-Schulz GEMMs, whose CTAs take an SM's shared
// memory and 13 warps of 112 registers but leave 18,944 registers, 51 warp slots and a sliver of shared
// memory unused.  A CTA of 256 threads at no more than 48 registers with no shared memory fits into that
// remainder, so one communication CTA per SM shares the SM with a GEMM CTA instead of taking the SM (and,
// for a two-CTA GEMM tile, its neighbour) away from the GEMM for as long as the transfer lasts.
#include "common.cuh"

namespace mmb {
namespace {

constexpr int MC_THREADS = 256;
constexpr int MC_UNROLL = 4;  // 16-byte requests in flight per thread

__device__ __forceinline__ uint4 mc_ld_reduce_bf16x8(const uint4* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_16(uint4* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

__global__ void __launch_bounds__(MC_THREADS)
mc_reduce_kernel(const uint4* __restrict__ mc_src, uint4* __restrict__ dst, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * MC_THREADS;
  long long i = static_cast<long long>(blockIdx.x) * MC_THREADS + threadIdx.x;
  for (; i + (MC_UNROLL - 1) * stride < n16; i += MC_UNROLL * stride) {
    uint4 v[MC_UNROLL];
#pragma unroll
    for (int u = 0; u < MC_UNROLL; ++u) v[u] = mc_ld_reduce_bf16x8(mc_src + i + u * stride);
#pragma unroll
    for (int u = 0; u < MC_UNROLL; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < n16; i += stride) dst[i] = mc_ld_reduce_bf16x8(mc_src + i);
}

__global__ void __launch_bounds__(MC_THREADS)
mc_broadcast_kernel(const uint4* __restrict__ src, uint4* __restrict__ mc_dst, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * MC_THREADS;
  long long i = static_cast<long long>(blockIdx.x) * MC_THREADS + threadIdx.x;
  for (; i + (MC_UNROLL - 1) * stride < n16; i += MC_UNROLL * stride) {
    uint4 v[MC_UNROLL];
#pragma unroll
    for (int u = 0; u < MC_UNROLL; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < MC_UNROLL; ++u) mc_st_16(mc_dst + i + u * stride, v[u]);
  }
  for (; i < n16; i += stride) mc_st_16(mc_dst + i, src[i]);
}

int check_args(const char* who, const void* a, const void* b, long long nbytes, int ctas) {
  MMB_REQUIRE(a != nullptr && b != nullptr, "%s: null pointer", who);
  MMB_REQUIRE(nbytes >= 0 && nbytes % 16 == 0, "%s: %lld bytes is not a multiple of 16", who, nbytes);
  MMB_REQUIRE(aligned16(a) && aligned16(b), "%s: pointers must be 16-byte aligned", who);
  MMB_REQUIRE(ctas >= 1 && ctas <= 1024, "%s: %d CTAs is outside 1..1024", who, ctas);
  return MMB_OK;
}

}  // namespace
}  // namespace mmb

extern "C" {

int mmb_multimem_reduce_bf16(const void* multicast_src, void* dst_dev, int64_t nbytes, int ctas, void* stream) {
  using namespace mmb;
  int rc = check_args("mmb_multimem_reduce_bf16", multicast_src, dst_dev, nbytes, ctas);
  if (rc != MMB_OK || nbytes == 0) return rc;
  mc_reduce_kernel<<<ctas, MC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(multicast_src), static_cast<uint4*>(dst_dev), nbytes / 16);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

int mmb_multimem_broadcast(const void* src_dev, void* multicast_dst, int64_t nbytes, int ctas, void* stream) {
  using namespace mmb;
  int rc = check_args("mmb_multimem_broadcast", src_dev, multicast_dst, nbytes, ctas);
  if (rc != MMB_OK || nbytes == 0) return rc;
  mc_broadcast_kernel<<<ctas, MC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src_dev), static_cast<uint4*>(multicast_dst), nbytes / 16);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

}  // extern "C"
