// Reduce-scatter and all-gather of the sharded optimizer step through NVSwitch multicast ("multimem").
//
// The multicast kernels work on a buffer that every GPU of the group has mapped at the same offset of one
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
//
// The peer kernels at the end of the file do the same two jobs with plain loads from and stores to the other
// GPUs' copies (peer pointers of the same symmetric buffers): per GPU (N-1)/N of the buffer crosses the links
// in each direction and collective, what a ring moves, in one hop and without taking SMs from the GEMMs.
// With two GPUs that is less than the multicast path moves (which sends a GPU's own copy through the switch
// as well).  Sums are formed in rank order with fp32 accumulation and rounded once.
#include "common.cuh"

namespace mmb {
namespace {

constexpr int MC_THREADS = 128;
constexpr int MC_UNROLL = 8;  // 16-byte requests in flight per thread

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

__global__ void __maxnreg__(64)
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

__global__ void __maxnreg__(64)
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


constexpr int MAX_PEERS = 16;
struct PeerPtrs {
  const uint4* p[MAX_PEERS];
};
struct PeerDsts {
  uint4* p[MAX_PEERS];
};

__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    acc[2 * j] += f.x;
    acc[2 * j + 1] += f.y;
  }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&acc)[8]) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  return o;
}

// dst[i] = bf16( sum over r = 0..W-1 of src_r[i] ), W copies of one range, U positions per thread in flight
template <int W, int U>
__global__ void __maxnreg__(64)
peer_reduce_kernel(PeerPtrs srcs, uint4* __restrict__ dst, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * MC_THREADS;
  long long i = static_cast<long long>(blockIdx.x) * MC_THREADS + threadIdx.x;
  for (; i + (U - 1) * stride < n16; i += U * stride) {
    uint4 v[U][W];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int r = 0; r < W; ++r) v[u][r] = __ldcs(srcs.p[r] + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < W; ++r) add_bf16x8(acc, v[u][r]);
      dst[i + u * stride] = pack_bf16x8(acc);
    }
  }
  for (; i < n16; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < W; ++r) add_bf16x8(acc, __ldcs(srcs.p[r] + i));
    dst[i] = pack_bf16x8(acc);
  }
}

// any group size up to MAX_PEERS: one position at a time, copies read in rank order
__global__ void __maxnreg__(64)
peer_reduce_any_kernel(PeerPtrs srcs, int world, uint4* __restrict__ dst, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * MC_THREADS;
  for (long long i = static_cast<long long>(blockIdx.x) * MC_THREADS + threadIdx.x; i < n16; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) add_bf16x8(acc, __ldcs(srcs.p[r] + i));
    dst[i] = pack_bf16x8(acc);
  }
}

// every dsts.p[r][i] = src[i] for the `count` destinations given (the caller leaves its own copy out)
__global__ void __maxnreg__(64)
peer_broadcast_kernel(const uint4* __restrict__ src, PeerDsts dsts, int count, long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * MC_THREADS;
  long long i = static_cast<long long>(blockIdx.x) * MC_THREADS + threadIdx.x;
  for (; i + (MC_UNROLL - 1) * stride < n16; i += MC_UNROLL * stride) {
    uint4 v[MC_UNROLL];
#pragma unroll
    for (int u = 0; u < MC_UNROLL; ++u) v[u] = src[i + u * stride];
    for (int r = 0; r < count; ++r) {
#pragma unroll
      for (int u = 0; u < MC_UNROLL; ++u) dsts.p[r][i + u * stride] = v[u];
    }
  }
  for (; i < n16; i += stride) {
    const uint4 v = src[i];
    for (int r = 0; r < count; ++r) dsts.p[r][i] = v;
  }
}

// An SM holds kernels of one shared-memory carve-out at a time: a kernel that asks for another one is
// admitted only after the SM has drained.  The GEMM CTAs need the largest carve-out, so these kernels ask
// for the same (they use no shared memory themselves).
void share_sm_with_gemm(const void* kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                       static_cast<int>(cudaSharedmemCarveoutMaxShared));
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
  share_sm_with_gemm(reinterpret_cast<const void*>(mc_reduce_kernel));
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
  share_sm_with_gemm(reinterpret_cast<const void*>(mc_broadcast_kernel));
  mc_broadcast_kernel<<<ctas, MC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src_dev), static_cast<uint4*>(multicast_dst), nbytes / 16);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

int mmb_peer_reduce_bf16(const void* const* copies, int world, void* dst_dev, int64_t nbytes, int ctas, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(copies != nullptr && world >= 1 && world <= MAX_PEERS, "mmb_peer_reduce_bf16: %d copies is outside 1..%d",
              world, MAX_PEERS);
  PeerPtrs srcs = {};
  for (int r = 0; r < world; ++r) {
    int rc = check_args("mmb_peer_reduce_bf16", copies[r], dst_dev, nbytes, ctas);
    if (rc != MMB_OK) return rc;
    srcs.p[r] = static_cast<const uint4*>(copies[r]);
  }
  if (nbytes == 0) return MMB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint4* dst = static_cast<uint4*>(dst_dev);
  const long long n16 = nbytes / 16;
  switch (world) {
    case 2:
      share_sm_with_gemm(reinterpret_cast<const void*>(peer_reduce_kernel<2, 4>));
      peer_reduce_kernel<2, 4><<<ctas, MC_THREADS, 0, st>>>(srcs, dst, n16);
      break;
    case 4:
      share_sm_with_gemm(reinterpret_cast<const void*>(peer_reduce_kernel<4, 2>));
      peer_reduce_kernel<4, 2><<<ctas, MC_THREADS, 0, st>>>(srcs, dst, n16);
      break;
    case 8:
      share_sm_with_gemm(reinterpret_cast<const void*>(peer_reduce_kernel<8, 1>));
      peer_reduce_kernel<8, 1><<<ctas, MC_THREADS, 0, st>>>(srcs, dst, n16);
      break;
    default:
      share_sm_with_gemm(reinterpret_cast<const void*>(peer_reduce_any_kernel));
      peer_reduce_any_kernel<<<ctas, MC_THREADS, 0, st>>>(srcs, world, dst, n16);
  }
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

int mmb_peer_broadcast(const void* src_dev, void* const* copies, int count, int64_t nbytes, int ctas, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(count >= 0 && count <= MAX_PEERS && (count == 0 || copies != nullptr),
              "mmb_peer_broadcast: %d destinations is outside 0..%d", count, MAX_PEERS);
  PeerDsts dsts = {};
  for (int r = 0; r < count; ++r) {
    int rc = check_args("mmb_peer_broadcast", src_dev, copies[r], nbytes, ctas);
    if (rc != MMB_OK) return rc;
    MMB_REQUIRE(copies[r] != src_dev, "mmb_peer_broadcast: destination %d is the source", r);
    dsts.p[r] = static_cast<uint4*>(copies[r]);
  }
  if (nbytes == 0 || count == 0) return MMB_OK;
  share_sm_with_gemm(reinterpret_cast<const void*>(peer_broadcast_kernel));
  peer_broadcast_kernel<<<ctas, MC_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src_dev), dsts, count, nbytes / 16);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

}  // extern "C"
