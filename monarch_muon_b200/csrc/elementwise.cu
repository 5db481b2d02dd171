// Bandwidth-bound multi-tensor kernels: the Muon weight update and the
// embedded AdamW.  Both take a table of tensors as kernel parameters and walk
// it with a grid-stride loop over 16-byte vectors, so one launch covers many
// parameter tensors without staging a pointer table in device memory.
#include "common.cuh"

namespace mmb {
namespace {

constexpr int THREADS = 256;
constexpr int MAX_SEG = 128;
constexpr int VEC = 8;  // elements per thread per step

// Round two values to the tensor's storage type and come back (models one torch op on each): one packed
// conversion instead of two (the conversion unit is the busiest pipe of the AdamW kernel).
template <typename T>
__device__ __forceinline__ void rd2(float& a, float& b);
template <>
__device__ __forceinline__ void rd2<__nv_bfloat16>(float& a, float& b) {
  const float2 f = __bfloat1622float2(__floats2bfloat162_rn(a, b));
  a = f.x;
  b = f.y;
}
template <>
__device__ __forceinline__ void rd2<float>(float&, float&) {}

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, bool vec, int n, float* out);
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, bool vec, int n, float* out) {
  if (vec) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = i < n ? __bfloat162float(p[i]) : 0.0f;
  }
}
template <>
__device__ __forceinline__ void load_vec<float>(const float* p, bool vec, int n, float* out) {
  if (vec) {
    float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = i < n ? p[i] : 0.0f;
  }
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, bool vec, int n, const float* in);
template <>
__device__ __forceinline__ void store_vec<__nv_bfloat16>(__nv_bfloat16* p, bool vec, int n, const float* in) {
  if (vec) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (i < n) p[i] = __float2bfloat16_rn(in[i]);
  }
}
template <>
__device__ __forceinline__ void store_vec<float>(float* p, bool vec, int n, const float* in) {
  if (vec) {
    reinterpret_cast<float4*>(p)[0] = make_float4(in[0], in[1], in[2], in[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(in[4], in[5], in[6], in[7]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (i < n) p[i] = in[i];
  }
}

// A table entry: tensors of one segment and where its vectors start in the
// launch-wide numbering.
struct UpdSeg {
  void* weight;
  const __nv_bfloat16* ortho;
  long long numel;
  int vec_ok;
};
struct UpdTable {
  UpdSeg seg[MAX_SEG];
  long long vec_start[MAX_SEG + 1];
  int nseg;
};

template <typename Tab>
__device__ __forceinline__ int find_segment(const Tab& tab, long long v) {
  int lo = 0, hi = tab.nseg;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (tab.vec_start[mid] <= v) lo = mid; else hi = mid;
  }
  return lo;
}

// W <- W + alpha*O, one fused multiply-add then one rounding to W's type, as
// torch's add_(other, alpha=) kernel does on a GPU.
template <typename WT>
__global__ void __launch_bounds__(THREADS)
muon_update_kernel(const __grid_constant__ UpdTable tab, float alpha) {
  const long long total = tab.vec_start[tab.nseg];
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < total; v += stride) {
    const int s = find_segment(tab, v);
    const UpdSeg& sg = tab.seg[s];
    const long long at = (v - tab.vec_start[s]) * VEC;
    const long long rem = sg.numel - at;
    const int n = rem >= VEC ? VEC : static_cast<int>(rem);
    const bool vec = sg.vec_ok && n == VEC;
    float w[VEC], o[VEC];
    WT* wp = static_cast<WT*>(sg.weight) + at;
    load_vec<WT>(wp, vec, n, w);
    load_vec<__nv_bfloat16>(sg.ortho + at, vec, n, o);
#pragma unroll
    for (int i = 0; i < VEC; ++i) w[i] = fmaf(alpha, o[i], w[i]);
    store_vec<WT>(wp, vec, n, w);
  }
}

struct AdamSeg {
  void* param;
  const void* grad;
  void* exp_avg;
  void* exp_avg_sq;
  long long numel;
  float inv_bc2_sqrt;  // 1 / sqrt(1 - beta2^step), formed in double: torch divides a CUDA tensor by a Python scalar
                       // by multiplying with the scalar's reciprocal
  float step_size;   // lr / (1 - beta1^step)
  int vec_ok;
  int pad_;
};
struct AdamTable {
  AdamSeg seg[MAX_SEG];
  long long vec_start[MAX_SEG + 1];
  int nseg;
};

// The reference issues one torch op per line (pretrain/src/models/monarch/
// monarch_muon.py:191-201); each op rounds to the tensor dtype, so `rd` is
// applied after every one of them.
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float* out) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// bf16 tensors, aligned full vectors: the four 16-byte loads of a thread's NEXT vector are issued before the
// current one is computed, so loads stay in flight during the ~70 instructions per element of arithmetic.
template <typename T>
__global__ void __launch_bounds__(THREADS, 4)
adamw_kernel(const __grid_constant__ AdamTable tab, float decay, float beta1, float one_m_beta1, float beta2,
             float one_m_beta2, float eps, const float* __restrict__ grad_scale_dev) {
  constexpr bool PREFETCH = sizeof(T) == 2;
  const float gscale = grad_scale_dev != nullptr ? *grad_scale_dev : 1.0f;
  const long long total = tab.vec_start[tab.nseg];
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  // where vector v lives, and (PREFETCH) its raw contents
  int s = 0, n = 0;
  long long at = 0;
  bool vec = false;
  uint4 rp = {}, rg = {}, rm = {}, rq = {};
  auto locate_and_fetch = [&](long long vv) {
    s = find_segment(tab, vv);
    const AdamSeg& sg = tab.seg[s];
    at = (vv - tab.vec_start[s]) * VEC;
    const long long rem = sg.numel - at;
    n = rem >= VEC ? VEC : static_cast<int>(rem);
    vec = sg.vec_ok && n == VEC;
    if (PREFETCH && vec) {
      rp = *reinterpret_cast<const uint4*>(static_cast<const T*>(sg.param) + at);
      rg = *reinterpret_cast<const uint4*>(static_cast<const T*>(sg.grad) + at);
      rm = *reinterpret_cast<const uint4*>(static_cast<const T*>(sg.exp_avg) + at);
      rq = *reinterpret_cast<const uint4*>(static_cast<const T*>(sg.exp_avg_sq) + at);
    }
  };
  if (v < total) locate_and_fetch(v);
  while (v < total) {
    const AdamSeg& sg = tab.seg[s];
    const bool cur_vec = vec;
    const int cur_n = n;
    const float inv_bc2_sqrt = sg.inv_bc2_sqrt, step_size = sg.step_size;
    T* pp = static_cast<T*>(sg.param) + at;
    T* mp = static_cast<T*>(sg.exp_avg) + at;
    T* vp = static_cast<T*>(sg.exp_avg_sq) + at;
    float p[VEC], g[VEC], m[VEC], q[VEC];
    if (PREFETCH && cur_vec) {
      unpack_bf16x8(rp, p);
      unpack_bf16x8(rg, g);
      unpack_bf16x8(rm, m);
      unpack_bf16x8(rq, q);
    } else {
      load_vec<T>(pp, cur_vec, cur_n, p);
      load_vec<T>(static_cast<const T*>(sg.grad) + at, cur_vec, cur_n, g);
      load_vec<T>(mp, cur_vec, cur_n, m);
      load_vec<T>(vp, cur_vec, cur_n, q);
    }
    v += stride;
    if (v < total) locate_and_fetch(v);   // from here on s, at, n, vec and the raw vectors describe the NEXT vector
    if (gscale != 1.0f) {
#pragma unroll
      for (int i = 0; i < VEC; i += 2) {  // like grad.mul_(coef) on the stored type
        g[i] = __fmul_rn(g[i], gscale);
        g[i + 1] = __fmul_rn(g[i + 1], gscale);
        rd2<T>(g[i], g[i + 1]);
      }
    }
    // two elements at a time so that every rounding to the tensor dtype is one packed conversion
#pragma unroll
    for (int i = 0; i < VEC; i += 2) {
      float p0 = p[i], p1 = p[i + 1];
      if (decay != 1.0f) {                                                      // p.mul_(1 - lr*wd)
        p0 = __fmul_rn(p0, decay); p1 = __fmul_rn(p1, decay);
        rd2<T>(p0, p1);
      }
      float m0 = __fmul_rn(m[i], beta1), m1 = __fmul_rn(m[i + 1], beta1);       // exp_avg.mul_(beta1)
      rd2<T>(m0, m1);
      m0 = fmaf(one_m_beta1, g[i], m0); m1 = fmaf(one_m_beta1, g[i + 1], m1);   // .add_(grad, alpha=1-beta1)
      rd2<T>(m0, m1);
      float v0 = __fmul_rn(q[i], beta2), v1 = __fmul_rn(q[i + 1], beta2);       // exp_avg_sq.mul_(beta2)
      rd2<T>(v0, v1);
      v0 = fmaf(one_m_beta2, __fmul_rn(g[i], g[i]), v0);                        // .addcmul_(grad, grad, value=1-beta2):
      v1 = fmaf(one_m_beta2, __fmul_rn(g[i + 1], g[i + 1]), v1);                //  a + value * (b * c), one fused multiply-add
      rd2<T>(v0, v1);
      float d0 = __fsqrt_rn(v0), d1 = __fsqrt_rn(v1);                           // exp_avg_sq.sqrt()
      rd2<T>(d0, d1);
      d0 = __fmul_rn(d0, inv_bc2_sqrt); d1 = __fmul_rn(d1, inv_bc2_sqrt);       // / sqrt(bc2): times the reciprocal
      rd2<T>(d0, d1);
      d0 = __fadd_rn(d0, eps); d1 = __fadd_rn(d1, eps);                         // .add_(eps)
      rd2<T>(d0, d1);
      p0 = fmaf(-step_size, __fdiv_rn(m0, d0), p0);                             // p.addcdiv_(m, denom, value=-lr/bc1)
      p1 = fmaf(-step_size, __fdiv_rn(m1, d1), p1);
      rd2<T>(p0, p1);
      p[i] = p0; p[i + 1] = p1; m[i] = m0; m[i + 1] = m1; q[i] = v0; q[i + 1] = v1;
    }
    store_vec<T>(pp, cur_vec, cur_n, p);
    store_vec<T>(mp, cur_vec, cur_n, m);
    store_vec<T>(vp, cur_vec, cur_n, q);
  }
}

// ---- global gradient norm and clip coefficient, without a host round trip
struct NormSeg {
  const void* grad;
  long long numel;
  int vec_ok;
  int pad_;
};
struct NormTable {
  NormSeg seg[MAX_SEG];
  long long vec_start[MAX_SEG + 1];
  int nseg;
};

// One partial sum of squares per CTA (fixed assignment of vectors to threads, tree reduction: reproducible).
template <typename T>
__global__ void __launch_bounds__(THREADS)
grad_sumsq_kernel(const __grid_constant__ NormTable tab, float* __restrict__ partials) {
  __shared__ float warp_sums[THREADS / 32];
  const long long total = tab.vec_start[tab.nseg];
  const long long stride = static_cast<long long>(gridDim.x) * THREADS;
  float acc = 0.0f;
  for (long long v = static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x; v < total; v += stride) {
    const int s = find_segment(tab, v);
    const NormSeg& sg = tab.seg[s];
    const long long at = (v - tab.vec_start[s]) * VEC;
    const long long rem = sg.numel - at;
    const int n = rem >= VEC ? VEC : static_cast<int>(rem);
    float g[VEC];
    load_vec<T>(static_cast<const T*>(sg.grad) + at, sg.vec_ok && n == VEC, n, g);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc = fmaf(g[i], g[i], acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) t += warp_sums[i];
    partials[blockIdx.x] += t;  // partials are zeroed by the caller; several launches accumulate
  }
}

// out[0] = sqrt(sum of partials), out[1] = min(1, max_norm / (out[0] + 1e-6))  (torch's clip_grad_norm_ rule)
__global__ void __launch_bounds__(THREADS)
clip_coef_kernel(const float* __restrict__ partials, int n, float max_norm, float* __restrict__ out) {
  __shared__ float warp_sums[THREADS / 32];
  float acc = 0.0f;
  for (int i = threadIdx.x; i < n; i += THREADS) acc += partials[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < THREADS / 32; ++i) t += warp_sums[i];
    const float norm = __fsqrt_rn(t);
    out[0] = norm;
    out[1] = fminf(1.0f, __fdiv_rn(max_norm, __fadd_rn(norm, 1e-6f)));
  }
}

int grid_for(long long total_vecs, int sms) {
  const int threads = stream_threads(THREADS);
  long long want = (total_vecs + threads - 1) / threads;
  long long cap = stream_grid_cap(sms);
  long long g = want < cap ? want : cap;
  return static_cast<int>(g < 1 ? 1 : g);
}

}  // namespace
}  // namespace mmb

extern "C" {

int mmb_muon_update(const mmb_update_seg* segs, int nseg, int weight_dtype, float alpha, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "mmb_muon_update: bad segment table");
  MMB_REQUIRE(weight_dtype == MMB_BF16 || weight_dtype == MMB_F32, "mmb_muon_update: weight_dtype %d", weight_dtype);
  if (nseg == 0) return MMB_OK;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_muon_update: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int base = 0; base < nseg; base += MAX_SEG) {
    UpdTable tab;
    tab.nseg = (nseg - base) < MAX_SEG ? (nseg - base) : MAX_SEG;
    long long vecs = 0;
    for (int i = 0; i < tab.nseg; ++i) {
      const mmb_update_seg& s = segs[base + i];
      MMB_REQUIRE(s.numel > 0 && s.weight && s.ortho, "mmb_muon_update: segment %d empty", base + i);
      tab.seg[i].weight = s.weight;
      tab.seg[i].ortho = static_cast<const __nv_bfloat16*>(s.ortho);
      tab.seg[i].numel = s.numel;
      tab.seg[i].vec_ok = aligned16(s.ortho) &&
                          ((reinterpret_cast<uintptr_t>(s.weight) & (weight_dtype == MMB_F32 ? 31u : 15u)) == 0);
      tab.vec_start[i] = vecs;
      vecs += (s.numel + VEC - 1) / VEC;
    }
    tab.vec_start[tab.nseg] = vecs;
    const int grid = grid_for(vecs, sms);
    if (weight_dtype == MMB_BF16)
      launch_stream_kernel(muon_update_kernel<__nv_bfloat16>, grid, THREADS, st, tab, alpha);
    else
      launch_stream_kernel(muon_update_kernel<float>, grid, THREADS, st, tab, alpha);
    MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  }
  return MMB_OK;
}

int64_t mmb_grad_norm_scratch_floats(void) {
  const int sms = mmb::sm_count();
  return static_cast<int64_t>(sms > 0 ? sms : 148) * 8 * 4;
}

int mmb_grad_norm_clip(const mmb_grad_seg* segs, int nseg, float max_norm, float* out_dev, float* scratch_dev,
                       int64_t scratch_floats, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "mmb_grad_norm_clip: bad segment table");
  MMB_REQUIRE(out_dev != nullptr && scratch_dev != nullptr, "mmb_grad_norm_clip: null output or scratch");
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_grad_norm_clip: no CUDA device");
  const int max_grid = sms * 8 * 4;
  MMB_REQUIRE(scratch_floats >= max_grid, "mmb_grad_norm_clip: scratch of %d floats needed, %lld given", max_grid,
              (long long)scratch_floats);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  MMB_CUDA_CHECK(cudaMemsetAsync(scratch_dev, 0, sizeof(float) * max_grid, st));
  // one table per dtype run of at most MAX_SEG tensors
  int base = 0;
  while (base < nseg) {
    const int dtype = segs[base].dtype;
    MMB_REQUIRE(dtype == MMB_BF16 || dtype == MMB_F32, "mmb_grad_norm_clip: dtype %d", dtype);
    NormTable tab;
    tab.nseg = 0;
    long long vecs = 0;
    while (base < nseg && tab.nseg < MAX_SEG && segs[base].dtype == dtype) {
      const mmb_grad_seg& s = segs[base];
      MMB_REQUIRE(s.numel > 0 && s.grad != nullptr, "mmb_grad_norm_clip: segment %d empty", base);
      NormSeg& d = tab.seg[tab.nseg];
      d.grad = s.grad;
      d.numel = s.numel;
      d.vec_ok = aligned16(s.grad);
      tab.vec_start[tab.nseg] = vecs;
      vecs += (s.numel + VEC - 1) / VEC;
      ++tab.nseg;
      ++base;
    }
    tab.vec_start[tab.nseg] = vecs;
    const int grid = grid_for(vecs, sms);
    if (dtype == MMB_BF16)
      grad_sumsq_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(tab, scratch_dev);
    else
      grad_sumsq_kernel<float><<<grid, THREADS, 0, st>>>(tab, scratch_dev);
    MMB_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  clip_coef_kernel<<<1, THREADS, 0, st>>>(scratch_dev, max_grid, max_norm, out_dev);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

int mmb_adamw_step(const mmb_adamw_seg* segs, int nseg, int dtype, double lr_in, double beta1_in, double beta2_in,
                   double weight_decay_in, double eps_in, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "mmb_adamw_step: bad segment table");
  MMB_REQUIRE(dtype == MMB_BF16 || dtype == MMB_F32, "mmb_adamw_step: dtype %d", dtype);
  if (nseg == 0) return MMB_OK;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_adamw_step: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Hyper-parameters arrive as doubles, the reference's Python floats; every derived scalar (1 - lr*wd,
  // 1 - beta, sqrt(1 - beta2^t), lr / (1 - beta1^t)) is formed in double as the reference forms it and
  // narrowed once to the fp32 the element-wise arithmetic runs in, as torch narrows a Python scalar.
  const double b1 = beta1_in, b2 = beta2_in, lrd = lr_in, wd = weight_decay_in;
  const float beta1 = static_cast<float>(b1), beta2 = static_cast<float>(b2), eps = static_cast<float>(eps_in);
  const float decay = wd > 0.0 ? static_cast<float>(1.0 - lrd * wd) : 1.0f;
  const uintptr_t amask = dtype == MMB_F32 ? 31u : 15u;
  for (int base = 0; base < nseg; base += MAX_SEG) {
    AdamTable tab;
    tab.nseg = (nseg - base) < MAX_SEG ? (nseg - base) : MAX_SEG;
    long long vecs = 0;
    for (int i = 0; i < tab.nseg; ++i) {
      const mmb_adamw_seg& s = segs[base + i];
      MMB_REQUIRE(s.numel > 0 && s.param && s.grad && s.exp_avg && s.exp_avg_sq, "mmb_adamw_step: segment %d empty",
                  base + i);
      MMB_REQUIRE(s.step >= 1, "mmb_adamw_step: segment %d has step %d (must be >= 1)", base + i, s.step);
      AdamSeg& d = tab.seg[i];
      d.param = s.param;
      d.grad = s.grad;
      d.exp_avg = s.exp_avg;
      d.exp_avg_sq = s.exp_avg_sq;
      d.numel = s.numel;
      double bc1 = 1.0 - pow(b1, static_cast<double>(s.step));
      double bc2 = 1.0 - pow(b2, static_cast<double>(s.step));
      d.inv_bc2_sqrt = static_cast<float>(1.0 / sqrt(bc2));
      d.step_size = static_cast<float>(lrd / bc1);
      d.vec_ok = (((reinterpret_cast<uintptr_t>(s.param) | reinterpret_cast<uintptr_t>(s.grad) |
                    reinterpret_cast<uintptr_t>(s.exp_avg) | reinterpret_cast<uintptr_t>(s.exp_avg_sq)) & amask) == 0);
      tab.vec_start[i] = vecs;
      vecs += (s.numel + VEC - 1) / VEC;
    }
    tab.vec_start[tab.nseg] = vecs;
    const int grid = grid_for(vecs, sms);
    const float omb1 = static_cast<float>(1.0 - b1), omb2 = static_cast<float>(1.0 - b2);
    if (dtype == MMB_BF16)
      launch_stream_kernel(adamw_kernel<__nv_bfloat16>, grid, THREADS, st, tab, decay, beta1, omb1, beta2, omb2, eps, device_grad_scale());
    else
      launch_stream_kernel(adamw_kernel<float>, grid, THREADS, st, tab, decay, beta1, omb1, beta2, omb2, eps, device_grad_scale());
    MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  }
  return MMB_OK;
}

}  // extern "C"
