// Batched quintic Newton-Schulz built from three fused GEMMs per iteration,
// plus the small kernels around it and a plain CUDA-core GEMM used only to
// cross-check the tensor-core path.
//
// For a block stored as rows x cols, let m = min(rows, cols), n = max.
// Per iteration (a, b, c = 3.4445, -4.7750, 2.0315):
//   Gram   A = X X^T                (m x m, contraction n)
//   Poly   P = b A + c A A          (m x m, contraction m; epilogue adds b A)
//   Apply  X = a X + P X            (m x n, contraction m; epilogue adds a X)
// Tall blocks (rows > cols) keep their stored orientation Y = X^T:
//   A = Y^T Y (both operands MN-major), Y = a Y + Y P.
// The Frobenius prescale s = 1/(||B||_F + 1e-7) is never applied to the data:
// the first Gram epilogue multiplies by s^2, the first Apply epilogue by s.
#include "common.cuh"

namespace mmb {

int gemm_tcgen05(const void* a, const void* b, const void* c, void* d, int batch, int M, int N, int K, int a_kmajor,
                 int b_kmajor, float alpha, float gamma, const float* inv_norm, int sigma_pow, int32_t* status,
                 cudaStream_t st);

namespace {

constexpr float NS_A = 3.4445f, NS_B = -4.7750f, NS_C = 2.0315f;
constexpr int NS_ITERS = 5;

// ------------------------------------------------------------ SIMT GEMM
// 64x64 output tile, 16-deep K slices, 256 threads x (4x4) results, fp32
// accumulation of bf16 inputs.  Operands are addressed through element strides
// so both storage orders go through the same code.
constexpr int ST = 64, SK = 16;

__global__ void __launch_bounds__(256)
simt_gemm_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                 const __nv_bfloat16* __restrict__ C, __nv_bfloat16* __restrict__ D, int M, int N, int K,
                 long long a_row, long long a_k, long long a_batch, long long b_row, long long b_k, long long b_batch,
                 float alpha, float gamma, const float* __restrict__ inv_norm, int sigma_pow) {
  __shared__ float As[SK][ST + 1];
  __shared__ float Bs[SK][ST + 1];
  const int b = blockIdx.z;
  const int m0 = blockIdx.y * ST, n0 = blockIdx.x * ST;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const __nv_bfloat16* Ab = A + b * a_batch;
  const __nv_bfloat16* Bb = B + b * b_batch;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += SK) {
    for (int i = threadIdx.x; i < ST * SK; i += 256) {
      // choose the index order that walks the contiguous dimension fastest
      int r, k;
      if (a_k == 1) { k = i % SK; r = i / SK; } else { r = i % ST; k = i / ST; }
      float v = 0.0f;
      if (m0 + r < M && k0 + k < K) v = __bfloat162float(Ab[(m0 + r) * a_row + (k0 + k) * a_k]);
      As[k][r] = v;
      if (b_k == 1) { k = i % SK; r = i / SK; } else { r = i % ST; k = i / ST; }
      v = 0.0f;
      if (n0 + r < N && k0 + k < K) v = __bfloat162float(Bb[(n0 + r) * b_row + (k0 + k) * b_k]);
      Bs[k][r] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SK; ++k) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = As[k][ty * 4 + i]; bv[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  float sigma = 1.0f;
  if (sigma_pow > 0 && inv_norm != nullptr) {
    float s = inv_norm[b];
    sigma = sigma_pow == 2 ? s * s : s;
  }
  const float sa = sigma * alpha, sg = sigma * gamma;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c >= N) continue;
      const long long at = (static_cast<long long>(b) * M + r) * N + c;
      const float addend = C != nullptr ? __bfloat162float(C[at]) : 0.0f;
      D[at] = __float2bfloat16_rn(fmaf(sa, acc[i][j], sg * addend));
    }
  }
}

int gemm_simt(const void* a, const void* b, const void* c, void* d, int batch, int M, int N, int K, int a_kmajor,
              int b_kmajor, float alpha, float gamma, const float* inv_norm, int sigma_pow, cudaStream_t st) {
  const long long a_row = a_kmajor ? K : 1, a_k = a_kmajor ? 1 : M;
  const long long b_row = b_kmajor ? K : 1, b_k = b_kmajor ? 1 : N;
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (batch - b0) < 65535 ? (batch - b0) : 65535;
    dim3 grid((N + ST - 1) / ST, (M + ST - 1) / ST, nb);
    const __nv_bfloat16* ap = static_cast<const __nv_bfloat16*>(a) + static_cast<long long>(b0) * M * K;
    const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(b) + static_cast<long long>(b0) * N * K;
    const __nv_bfloat16* cp = c ? static_cast<const __nv_bfloat16*>(c) + static_cast<long long>(b0) * M * N : nullptr;
    __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(d) + static_cast<long long>(b0) * M * N;
    simt_gemm_kernel<<<grid, 256, 0, st>>>(ap, bp, cp, dp, M, N, K, a_row, a_k, static_cast<long long>(M) * K, b_row,
                                          b_k, static_cast<long long>(N) * K, alpha, gamma,
                                          inv_norm ? inv_norm + b0 : nullptr, sigma_pow);
    MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  }
  return MMB_OK;
}

int gemm_dispatch(int backend, const void* a, const void* b, const void* c, void* d, int batch, int M, int N, int K,
                  int a_kmajor, int b_kmajor, float alpha, float gamma, const float* inv_norm, int sigma_pow,
                  int32_t* status, cudaStream_t st) {
  if (backend == MMB_NS_TCGEN05)
    return gemm_tcgen05(a, b, c, d, batch, M, N, K, a_kmajor, b_kmajor, alpha, gamma, inv_norm, sigma_pow, status, st);
  if (backend == MMB_NS_SIMT)
    return gemm_simt(a, b, c, d, batch, M, N, K, a_kmajor, b_kmajor, alpha, gamma, inv_norm, sigma_pow, st);
  return fail(MMB_ERR_INVALID, "unknown Newton-Schulz backend %d", backend);
}

// --------------------------------------------------- norms (one CTA per block)
// sum of squares of a bf16 block, fixed summation order
__global__ void __launch_bounds__(256)
block_sumsq_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long block_elems, float* __restrict__ out) {
  __shared__ float warp_sums[8];
  const __nv_bfloat16* p = x + static_cast<long long>(blockIdx.x) * block_elems;
  float acc = 0.0f;
  const bool vec = (block_elems % 8 == 0) && ((reinterpret_cast<uintptr_t>(p) & 15u) == 0);
  if (vec) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
    for (long long i = threadIdx.x; i < block_elems / 8; i += 256) {
      uint4 v = p4[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
      }
    }
  } else {
    for (long long i = threadIdx.x; i < block_elems; i += 256) {
      float f = __bfloat162float(p[i]);
      acc = fmaf(f, f, acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += warp_sums[i];
    out[blockIdx.x] = t;
  }
}

// s = 1 / (sqrt(sumsq) + 1e-7): the reference adds eps to the norm, not under the root
__global__ void inv_norm_kernel(const float* __restrict__ sumsq, float* __restrict__ inv, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) inv[i] = __fdiv_rn(1.0f, __fadd_rn(__fsqrt_rn(sumsq[i]), 1e-7f));
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct NsLayout {
  size_t gram, poly, xa, xb, inv, sumsq, total;
};

NsLayout ns_layout(int batch, int rows, int cols) {
  const size_t m = rows < cols ? rows : cols;
  const size_t blk = static_cast<size_t>(rows) * cols;
  NsLayout l;
  size_t at = 0;
  l.gram = at; at = align_up(at + static_cast<size_t>(batch) * m * m * 2, 1024);
  l.poly = at; at = align_up(at + static_cast<size_t>(batch) * m * m * 2, 1024);
  l.xa = at;   at = align_up(at + static_cast<size_t>(batch) * blk * 2, 1024);
  l.xb = at;   at = align_up(at + static_cast<size_t>(batch) * blk * 2, 1024);
  l.inv = at;  at = align_up(at + static_cast<size_t>(batch) * 4, 1024);
  l.sumsq = at; at = align_up(at + static_cast<size_t>(batch) * 4, 1024);
  l.total = at;
  return l;
}

}  // namespace
}  // namespace mmb

extern "C" {

int64_t mmb_ns_workspace_bytes(int batch, int rows, int cols) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  return static_cast<int64_t>(mmb::ns_layout(batch, rows, cols).total);
}

int mmb_gemm_bf16(const void* a_dev, const void* b_dev, const void* c_dev, void* d_dev, int batch, int M, int N, int K,
                  int a_kmajor, int b_kmajor, float alpha, float gamma, const float* inv_norm_dev, int sigma_pow,
                  int backend, int32_t* status_dev, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(a_dev && b_dev && d_dev, "mmb_gemm_bf16: null operand");
  MMB_REQUIRE(batch > 0 && M > 0 && N > 0 && K > 0, "mmb_gemm_bf16: bad shape %d x (%d,%d,%d)", batch, M, N, K);
  MMB_REQUIRE(sigma_pow >= 0 && sigma_pow <= 2, "mmb_gemm_bf16: sigma_pow %d", sigma_pow);
  return gemm_dispatch(backend, a_dev, b_dev, c_dev, d_dev, batch, M, N, K, a_kmajor, b_kmajor, alpha, gamma,
                       inv_norm_dev, sigma_pow, status_dev, static_cast<cudaStream_t>(stream));
}

int mmb_newton_schulz(const void* x_dev, void* out_dev, const float* block_sumsq_dev, int batch, int rows, int cols,
                      void* workspace_dev, int64_t workspace_bytes, int backend, int32_t* status_dev, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(x_dev && out_dev && workspace_dev, "mmb_newton_schulz: null pointer");
  MMB_REQUIRE(batch > 0 && rows > 0 && cols > 0, "mmb_newton_schulz: bad shape (%d,%d,%d)", batch, rows, cols);
  MMB_REQUIRE((reinterpret_cast<uintptr_t>(workspace_dev) & 1023u) == 0, "mmb_newton_schulz: workspace not 1 KiB aligned");
  const NsLayout l = ns_layout(batch, rows, cols);
  MMB_REQUIRE(workspace_bytes >= static_cast<int64_t>(l.total), "mmb_newton_schulz: workspace %lld < %lld bytes",
              (long long)workspace_bytes, (long long)l.total);
  if (backend == MMB_NS_TCGEN05)
    MMB_REQUIRE(rows % 8 == 0 && cols % 8 == 0, "mmb_newton_schulz: tensor-core path needs rows, cols multiples of 8");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace_dev);
  __nv_bfloat16* gram = reinterpret_cast<__nv_bfloat16*>(ws + l.gram);
  __nv_bfloat16* poly = reinterpret_cast<__nv_bfloat16*>(ws + l.poly);
  __nv_bfloat16* xa = reinterpret_cast<__nv_bfloat16*>(ws + l.xa);
  __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(ws + l.xb);
  float* inv = reinterpret_cast<float*>(ws + l.inv);
  float* sumsq = reinterpret_cast<float*>(ws + l.sumsq);

  const float* ss = block_sumsq_dev;
  if (ss == nullptr) {
    block_sumsq_bf16_kernel<<<batch, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x_dev),
                                                   static_cast<long long>(rows) * cols, sumsq);
    MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
    ss = sumsq;
  }
  inv_norm_kernel<<<(batch + 255) / 256, 256, 0, st>>>(ss, inv, batch);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();

  const bool tall = rows > cols;
  const int m = tall ? cols : rows;
  const int n = tall ? rows : cols;
  const __nv_bfloat16* cur = static_cast<const __nv_bfloat16*>(x_dev);
  for (int it = 0; it < NS_ITERS; ++it) {
    __nv_bfloat16* nxt = (it == NS_ITERS - 1) ? static_cast<__nv_bfloat16*>(out_dev) : ((it & 1) ? xb : xa);
    const int first = it == 0;
    int rc;
    // Gram: wide X X^T (both K-major, K = n); tall Y^T Y (both MN-major, K = n = rows)
    rc = gemm_dispatch(backend, cur, cur, nullptr, gram, batch, m, m, n, tall ? 0 : 1, tall ? 0 : 1, 1.0f, 0.0f, inv,
                       first ? 2 : 0, status_dev, st);
    if (rc != MMB_OK) return rc;
    // Poly: P = b A + c A A (A symmetric, so A serves as the K-major second operand)
    rc = gemm_dispatch(backend, gram, gram, gram, poly, batch, m, m, m, 1, 1, NS_C, NS_B, nullptr, 0, status_dev, st);
    if (rc != MMB_OK) return rc;
    // Apply: wide X' = a X + P X  (opA = P K-major, opB = X stored [K][N] -> MN-major)
    //        tall Y' = a Y + Y P  (opA = Y K-major, opB = P K-major by symmetry)
    if (!tall)
      rc = gemm_dispatch(backend, poly, cur, cur, nxt, batch, m, n, m, 1, 0, 1.0f, NS_A, inv, first ? 1 : 0, status_dev, st);
    else
      rc = gemm_dispatch(backend, cur, poly, cur, nxt, batch, n, m, m, 1, 1, 1.0f, NS_A, inv, first ? 1 : 0, status_dev, st);
    if (rc != MMB_OK) return rc;
    cur = nxt;
  }
  return MMB_OK;
}

}  // extern "C"
