// Batched quintic Newton-Schulz built from three fused GEMMs per iteration,
// plus the small kernels around it and a plain CUDA-core GEMM used only to
// cross-check the tensor-core path.
//
// For a block stored as rows x cols, let m = min(rows, cols), n = max.  With
// (a, b, c) = (3.4445, -4.7750, 2.0315) the reference iterates
//   A = X X^T ;  X <- a X + b A X + c A A X = (a I + b A + c A^2) X.
// Completing the square, a I + b A + c A^2 = c (A + beta I)^2 + kappa I with
// beta = b / (2c) and kappa = a - b^2 / (4c), so one iteration is three GEMMs
// whose epilogues only scale, add a constant on the diagonal and round:
//   Gram   Ah = X X^T + beta I            (m x m, contraction n, symmetric)
//   Poly   Pp = c Ah Ah + kappa I         (m x m, contraction m, symmetric)
//   Apply  X  = Pp X                      (m x n, contraction m)
// The sum c(.)^2 + kappa has only positive terms, so it is better conditioned
// than a + b s + c s^2 evaluated term by term.  Symmetric results are stored
// and read block-upper only (see gemm_tcgen05.cu).
// Tall blocks (rows > cols) keep their stored orientation Y = X^T:
//   Ah = Y^T Y + beta I (both operands MN-major), Y = Y Pp.
// The Frobenius prescale s = 1/(||B||_F + 1e-7) is never applied to the data:
// the first Gram epilogue multiplies by s^2, the first Apply epilogue by s.
#include "common.cuh"
#include "gemm.cuh"

namespace mmb {

namespace {

constexpr double NS_A = 3.4445, NS_B = -4.7750, NS_C = 2.0315;
constexpr int NS_ITERS = 5;

// ------------------------------------------------------------ SIMT GEMM
// 64x64 output tile, 16-deep K slices, 256 threads x (4x4) results, fp32
// accumulation of bf16 inputs; same operand modes and output convention as
// the tensor-core kernel.
constexpr int ST = 64, SK = 16;

__device__ __forceinline__ float fetch(const __nv_bfloat16* base, int mode, int rows, int K, int r, int k) {
  if (r >= rows || k >= K) return 0.0f;
  bool kmajor = mode == GEMM_K || (mode == GEMM_SYM && (r >> 8) <= (k >> 8));
  if (mode == GEMM_SYM && !kmajor) return __bfloat162float(base[static_cast<long long>(k) * rows + r]);  // mirror
  if (mode == GEMM_MN) return __bfloat162float(base[static_cast<long long>(k) * rows + r]);
  return __bfloat162float(base[static_cast<long long>(r) * K + k]);
}

__global__ void __launch_bounds__(256)
simt_gemm_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                 __nv_bfloat16* __restrict__ D, int M, int N, int K, int a_mode, int b_mode, int sym_out, float alpha,
                 float diag, const float* __restrict__ inv_norm, int sigma_pow) {
  __shared__ float As[SK][ST + 1];
  __shared__ float Bs[SK][ST + 1];
  const int b = blockIdx.z;
  const int m0 = blockIdx.y * ST, n0 = blockIdx.x * ST;
  if (sym_out && (m0 >> 8) > (n0 >> 8)) return;  // below the block diagonal: not stored
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const __nv_bfloat16* Ab = A + static_cast<long long>(b) * M * K;
  const __nv_bfloat16* Bb = B + static_cast<long long>(b) * N * K;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += SK) {
    for (int i = threadIdx.x; i < ST * SK; i += 256) {
      int r, k;
      if (a_mode == GEMM_K) { k = i % SK; r = i / SK; } else { r = i % ST; k = i / ST; }
      As[k][r] = fetch(Ab, a_mode, M, K, m0 + r, k0 + k);
      if (b_mode == GEMM_K) { k = i % SK; r = i / SK; } else { r = i % ST; k = i / ST; }
      Bs[k][r] = fetch(Bb, b_mode, N, K, n0 + r, k0 + k);
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
  const float scale = sigma * alpha;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c >= N) continue;
      float x = scale * acc[i][j];
      if (r == c) x += diag;
      D[(static_cast<long long>(b) * M + r) * N + c] = __float2bfloat16_rn(x);
    }
  }
}

}  // namespace

int gemm_simt(const GemmCall& g, cudaStream_t st) {
  for (int b0 = 0; b0 < g.batch; b0 += 65535) {
    const int nb = (g.batch - b0) < 65535 ? (g.batch - b0) : 65535;
    dim3 grid((g.N + ST - 1) / ST, (g.M + ST - 1) / ST, nb);
    const __nv_bfloat16* ap = static_cast<const __nv_bfloat16*>(g.a) + static_cast<long long>(b0) * g.M * g.K;
    const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(g.b) + static_cast<long long>(b0) * g.N * g.K;
    __nv_bfloat16* dp = static_cast<__nv_bfloat16*>(g.d) + static_cast<long long>(b0) * g.M * g.N;
    simt_gemm_kernel<<<grid, 256, 0, st>>>(ap, bp, dp, g.M, g.N, g.K, g.a_mode, g.b_mode, g.sym_out, g.alpha, g.diag,
                                          g.inv_norm ? g.inv_norm + b0 : nullptr, g.sigma_pow);
    MMB_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  return MMB_OK;
}

namespace {

int gemm_dispatch(int backend, const GemmCall& g, int32_t* status, cudaStream_t st) {
  if (backend == MMB_NS_TCGEN05 || backend == MMB_NS_TCGEN05_MULTI) return gemm_tcgen05(g, status, st);
  if (backend == MMB_NS_SIMT) return gemm_simt(g, st);
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

// W[b] <- W[b] + alpha * O[b] for blocks reached through a pointer table: the update that follows
// Newton-Schulz when it is not fused into the last GEMM's epilogue (cross-check back end).
template <typename WT>
__global__ void __launch_bounds__(256)
update_blocks_kernel(void* const* __restrict__ w_ptrs, const __nv_bfloat16* __restrict__ ortho, long long block_elems,
                     float alpha) {
  WT* w = static_cast<WT*>(w_ptrs[blockIdx.y]);
  const __nv_bfloat16* o = ortho + static_cast<long long>(blockIdx.y) * block_elems;
  for (long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; i < block_elems;
       i += static_cast<long long>(gridDim.x) * 256) {
    const float x = fmaf(alpha, __bfloat162float(o[i]), static_cast<float>(w[i]));
    w[i] = static_cast<WT>(x);
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct NsLayout {
  size_t gram, poly, xa, xb, inv, sumsq, sched, total;
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
  l.sched = at; at += 1024;  // counters of the dynamic tile schedule
  l.total = at;
  return l;
}

}  // namespace
}  // namespace mmb

extern "C" {

int mmb_gemm_occupancy(int pair, int* out) { return mmb::gemm_occupancy(pair, out); }

int64_t mmb_ns_workspace_bytes(int batch, int rows, int cols) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  return static_cast<int64_t>(mmb::ns_layout(batch, rows, cols).total);
}

int mmb_gemm_bf16(const void* a_dev, const void* b_dev, void* d_dev, int batch, int M, int N, int K, int a_mode,
                  int b_mode, int sym_out, float alpha, float diag, const float* inv_norm_dev, int sigma_pow,
                  int backend, int32_t* status_dev, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(a_dev && b_dev && d_dev, "mmb_gemm_bf16: null operand");
  MMB_REQUIRE(batch > 0 && M > 0 && N > 0 && K > 0, "mmb_gemm_bf16: bad shape %d x (%d,%d,%d)", batch, M, N, K);
  MMB_REQUIRE(sigma_pow >= 0 && sigma_pow <= 2, "mmb_gemm_bf16: sigma_pow %d", sigma_pow);
  MMB_REQUIRE(a_mode >= 0 && a_mode <= 2 && b_mode >= 0 && b_mode <= 2, "mmb_gemm_bf16: operand mode");
  GemmCall g{a_dev, b_dev, d_dev, batch, M, N, K, a_mode, b_mode, sym_out, alpha, diag, inv_norm_dev, sigma_pow};
  return gemm_dispatch(backend, g, status_dev, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

namespace mmb {
namespace {

// Newton-Schulz on `batch` blocks.  With w_ptrs == nullptr the result goes to out_dev; otherwise out_dev is
// not used and the result updates the blocks' weights, W[b] <- W[b] + alpha * NS(X)[b].
int newton_schulz_impl(const char* who, const void* x_dev, void* out_dev, const float* block_sumsq_dev, int batch,
                       int rows, int cols, void* workspace_dev, int64_t workspace_bytes, int backend,
                       int32_t* status_dev, void* stream, void* const* w_ptrs, int w_f32, float alpha) {
  MMB_REQUIRE(x_dev && (out_dev || w_ptrs) && workspace_dev, "%s: null pointer", who);
  MMB_REQUIRE(batch > 0 && rows > 0 && cols > 0, "%s: bad shape (%d,%d,%d)", who, batch, rows, cols);
  MMB_REQUIRE((reinterpret_cast<uintptr_t>(workspace_dev) & 1023u) == 0, "%s: workspace not 1 KiB aligned", who);
  const NsLayout l = ns_layout(batch, rows, cols);
  MMB_REQUIRE(workspace_bytes >= static_cast<int64_t>(l.total), "%s: workspace %lld < %lld bytes", who,
              (long long)workspace_bytes, (long long)l.total);
  if (backend == MMB_NS_TCGEN05 || backend == MMB_NS_TCGEN05_MULTI)
    MMB_REQUIRE(rows % 8 == 0 && cols % 8 == 0, "%s: tensor-core path needs rows, cols multiples of 8", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace_dev);
  __nv_bfloat16* gram = reinterpret_cast<__nv_bfloat16*>(ws + l.gram);
  __nv_bfloat16* poly = reinterpret_cast<__nv_bfloat16*>(ws + l.poly);
  __nv_bfloat16* xa = reinterpret_cast<__nv_bfloat16*>(ws + l.xa);
  __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(ws + l.xb);
  float* inv = reinterpret_cast<float*>(ws + l.inv);
  float* sumsq = reinterpret_cast<float*>(ws + l.sumsq);
  int* sched = nullptr;
  if ((backend == MMB_NS_TCGEN05 || backend == MMB_NS_TCGEN05_MULTI) && gemm_schedule_dynamic()) {
    sched = reinterpret_cast<int*>(ws + l.sched);
    MMB_CUDA_CHECK(cudaMemsetAsync(sched, 0, 2 * sizeof(int), st));  // each launch leaves them at zero again
  }

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

  const float beta = static_cast<float>(NS_B / (2.0 * NS_C));
  const float kappa = static_cast<float>(NS_A - NS_B * NS_B / (4.0 * NS_C));
  const float c = static_cast<float>(NS_C);
  const bool tall = rows > cols;
  const int m = tall ? cols : rows;
  const int n = tall ? rows : cols;
  if (backend == MMB_NS_TCGEN05 && ns_onchip_fits(rows, cols))   // the whole iteration in one launch, on chip
    return ns_onchip(x_dev, out_dev, inv, batch, rows, cols, beta, kappa, c, w_ptrs, w_f32, alpha, status_dev, st);
  if (backend == MMB_NS_TCGEN05_MULTI) backend = MMB_NS_TCGEN05;
  const __nv_bfloat16* cur = static_cast<const __nv_bfloat16*>(x_dev);
  const bool fuse_update = w_ptrs != nullptr && backend == MMB_NS_TCGEN05;
  for (int it = 0; it < NS_ITERS; ++it) {
    const bool last = it == NS_ITERS - 1;
    __nv_bfloat16* nxt = (last && w_ptrs == nullptr) ? static_cast<__nv_bfloat16*>(out_dev) : ((it & 1) ? xb : xa);
    const int first = it == 0;
    int rc;
    // Gram: wide X X^T (K-major operands, contraction n); tall Y^T Y (MN-major operands, contraction rows)
    const int xmode = tall ? GEMM_MN : GEMM_K;
    GemmCall gram_call{cur, cur, gram, batch, m, m, n, xmode, xmode, 1, 1.0f, beta, inv, first ? 2 : 0, sched};
    if ((rc = gemm_dispatch(backend, gram_call, status_dev, st)) != MMB_OK) return rc;
    // Poly: Pp = c Ah Ah + kappa I
    GemmCall poly_call{gram, gram, poly, batch, m, m, m, GEMM_SYM, GEMM_SYM, 1, c, kappa, nullptr, 0, sched};
    if ((rc = gemm_dispatch(backend, poly_call, status_dev, st)) != MMB_OK) return rc;
    // Apply: wide X' = Pp X (B = X stored [K][N]); tall Y' = Y Pp (A = Y, B = Pp by symmetry)
    GemmCall ap = !tall ? GemmCall{poly, cur, nxt, batch, m, n, m, GEMM_SYM, GEMM_MN, 0, 1.0f, 0.0f, inv, first ? 1 : 0, sched}
                        : GemmCall{cur, poly, nxt, batch, n, m, m, GEMM_K, GEMM_SYM, 0, 1.0f, 0.0f, inv, first ? 1 : 0, sched};
    if (last && fuse_update) {  // the result (rows x cols, stored orientation) never reaches memory
      ap.upd_w = w_ptrs;
      ap.upd_alpha = alpha;
      ap.upd_f32 = w_f32;
    }
    if ((rc = gemm_dispatch(backend, ap, status_dev, st)) != MMB_OK) return rc;
    cur = nxt;
  }
  if (w_ptrs != nullptr && !fuse_update) {
    const long long blk = static_cast<long long>(rows) * cols;
    long long gx = (blk + 255) / 256;
    if (gx > 64) gx = 64;
    for (int b0 = 0; b0 < batch; b0 += 65535) {
      const int nb = (batch - b0) < 65535 ? (batch - b0) : 65535;
      dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(nb));
      if (w_f32)
        update_blocks_kernel<float><<<grid, 256, 0, st>>>(w_ptrs + b0, cur + b0 * blk, blk, alpha);
      else
        update_blocks_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(w_ptrs + b0, cur + b0 * blk, blk, alpha);
      MMB_CUDA_CHECK(cudaGetLastError());
      count_launch();
    }
  }
  return MMB_OK;
}

}  // namespace
}  // namespace mmb

extern "C" {

int mmb_newton_schulz(const void* x_dev, void* out_dev, const float* block_sumsq_dev, int batch, int rows, int cols,
                      void* workspace_dev, int64_t workspace_bytes, int backend, int32_t* status_dev, void* stream) {
  return mmb::newton_schulz_impl("mmb_newton_schulz", x_dev, out_dev, block_sumsq_dev, batch, rows, cols, workspace_dev,
                                 workspace_bytes, backend, status_dev, stream, nullptr, 0, 0.0f);
}

int mmb_newton_schulz_update(const void* x_dev, const float* block_sumsq_dev, int batch, int rows, int cols,
                             void* const* weight_ptrs_dev, int weight_dtype, float alpha, void* workspace_dev,
                             int64_t workspace_bytes, int backend, int32_t* status_dev, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(weight_ptrs_dev != nullptr, "mmb_newton_schulz_update: null weight pointer table");
  MMB_REQUIRE(weight_dtype == MMB_BF16 || weight_dtype == MMB_F32, "mmb_newton_schulz_update: weight_dtype %d",
              weight_dtype);
  return newton_schulz_impl("mmb_newton_schulz_update", x_dev, nullptr, block_sumsq_dev, batch, rows, cols, workspace_dev,
                            workspace_bytes, backend, status_dev, stream, weight_ptrs_dev, weight_dtype == MMB_F32, alpha);
}

int mmb_wait_probe(int64_t limit_cycles, int32_t* status_dev, void* stream) {
  return mmb::wait_probe(limit_cycles, status_dev, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
