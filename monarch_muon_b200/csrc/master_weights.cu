// Steps on fp32 master weights with a bf16 copy for the model: the fine-tuning
// optimizer of the reference keeps `master` (fp32), updates it, then writes
// `p.copy_(master)` (finetune/sft_optimizer.py:33-59).  Here the update and the
// down-cast are one pass: read master (4 B), read the update's inputs, write
// master (4 B) and the bf16 parameter (2 B).
//
//   mmb_muon_update_master : master += alpha * O          (sft_optimizer.py:48-49)
//   mmb_adamw_master_step  : torch.optim AdamW on master  (sft_optimizer.py:51-55)
#include <cmath>

#include "common.cuh"

namespace mmb {
namespace {

constexpr int THREADS = 256;
constexpr int MAX_SEG = 96;
constexpr int VEC = 8;  // elements per thread per step

__device__ __forceinline__ void load8(const float* p, bool vec, int n, float* out) {
  if (vec) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = i < n ? p[i] : 0.0f;
  }
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, bool vec, int n, float* out) {
  if (vec) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = i < n ? __bfloat162float(p[i]) : 0.0f;
  }
}
__device__ __forceinline__ void store8(float* p, bool vec, int n, const float* in) {
  if (vec) {
    reinterpret_cast<float4*>(p)[0] = make_float4(in[0], in[1], in[2], in[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(in[4], in[5], in[6], in[7]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (i < n) p[i] = in[i];
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, bool vec, int n, const float* in) {
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

struct Seg {
  float* master;
  __nv_bfloat16* shadow;   // may be null
  const void* a;           // update: O (bf16); AdamW: gradient (grad dtype)
  float* exp_avg;          // AdamW only
  float* exp_avg_sq;
  long long numel;
  int step;                // AdamW: the already incremented step count
  int vec_ok;
};
struct Table {
  Seg seg[MAX_SEG];
  long long vec_start[MAX_SEG + 1];
  int nseg;
};

__device__ __forceinline__ int find_segment(const Table& tab, long long v) {
  int lo = 0, hi = tab.nseg;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tab.vec_start[mid] <= v) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(THREADS)
update_master_kernel(const __grid_constant__ Table tab, float alpha) {
  const long long total = tab.vec_start[tab.nseg];
  const long long stride = static_cast<long long>(gridDim.x) * THREADS;
  for (long long v = static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x; v < total; v += stride) {
    const int s = find_segment(tab, v);
    const Seg& sg = tab.seg[s];
    const long long at = (v - tab.vec_start[s]) * VEC;
    const long long rem = sg.numel - at;
    const int n = rem >= VEC ? VEC : static_cast<int>(rem);
    const bool vec = sg.vec_ok && n == VEC;
    float w[VEC], o[VEC];
    load8(sg.master + at, vec, n, w);
    load8(static_cast<const __nv_bfloat16*>(sg.a) + at, vec, n, o);
#pragma unroll
    for (int i = 0; i < VEC; ++i) w[i] = fmaf(alpha, o[i], w[i]);   // master.add_(update, alpha=alpha)
    store8(sg.master + at, vec, n, w);
    if (sg.shadow != nullptr) store8(sg.shadow + at, vec, n, w);    // p.copy_(master)
  }
}

// The AdamW update the reference's fine-tuning optimizer runs on a GPU: torch.optim's FUSED kernel
// (finetune/sft_optimizer.py:52-55 passes fused=p.is_cuda), on the fp32 master.  That kernel works in fp32
// throughout, hyper-parameters included: 1 - beta is formed from the float beta, the bias corrections
// 1 - beta^step by the float power function, and its multiply-adds contract as below (each line checked
// against torch._fused_adamw_ on 2^20 elements: equal bit for bit).
template <typename GradT>
__global__ void __launch_bounds__(THREADS)
adamw_master_kernel(const __grid_constant__ Table tab, float lr, float weight_decay, float beta1, float beta2, float eps) {
  const long long total = tab.vec_start[tab.nseg];
  const long long stride = static_cast<long long>(gridDim.x) * THREADS;
  const float a1 = __fsub_rn(1.0f, beta1), a2 = __fsub_rn(1.0f, beta2);
  const float lw = __fmul_rn(lr, weight_decay);
  int cached_step = -1;
  float bc2_sqrt = 1.0f, step_size = 0.0f;
  for (long long v = static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x; v < total; v += stride) {
    const int s = find_segment(tab, v);
    const Seg& sg = tab.seg[s];
    if (sg.step != cached_step) {   // bias corrections as the fused kernel forms them, on the device, in fp32
      cached_step = sg.step;
      const float t = static_cast<float>(sg.step);
      const float bc1 = __fsub_rn(1.0f, powf(beta1, t));
      bc2_sqrt = __fsqrt_rn(__fsub_rn(1.0f, powf(beta2, t)));
      step_size = __fdiv_rn(lr, bc1);
    }
    const long long at = (v - tab.vec_start[s]) * VEC;
    const long long rem = sg.numel - at;
    const int n = rem >= VEC ? VEC : static_cast<int>(rem);
    const bool vec = sg.vec_ok && n == VEC;
    float p[VEC], g[VEC], m[VEC], q[VEC];
    load8(sg.master + at, vec, n, p);
    load8(static_cast<const GradT*>(sg.a) + at, vec, n, g);
    load8(sg.exp_avg + at, vec, n, m);
    load8(sg.exp_avg_sq + at, vec, n, q);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float pi = weight_decay != 0.0f ? fmaf(-lw, p[i], p[i]) : p[i];            // param -= lr * weight_decay * param
      const float mi = fmaf(beta1, m[i], __fmul_rn(a1, g[i]));                   // exp_avg = beta1 * exp_avg + (1 - beta1) * grad
      const float vi = fmaf(beta2, q[i], __fmul_rn(a2, __fmul_rn(g[i], g[i])));  // exp_avg_sq = beta2 * exp_avg_sq + (1 - beta2) * grad * grad
      const float d = __fadd_rn(__fdiv_rn(__fsqrt_rn(vi), bc2_sqrt), eps);       // denom = sqrt(exp_avg_sq) / bias_correction2_sqrt + eps
      pi = __fsub_rn(pi, __fdiv_rn(__fmul_rn(step_size, mi), d));                // param -= step_size * exp_avg / denom
      p[i] = pi; m[i] = mi; q[i] = vi;
    }
    store8(sg.master + at, vec, n, p);
    store8(sg.exp_avg + at, vec, n, m);
    store8(sg.exp_avg_sq + at, vec, n, q);
    if (sg.shadow != nullptr) store8(sg.shadow + at, vec, n, p);
  }
}

int grid_for(long long total_vecs, int sms) {
  const long long want = (total_vecs + THREADS - 1) / THREADS;
  const long long cap = stream_grid_cap(sms);
  const long long g = want < cap ? want : cap;
  return static_cast<int>(g < 1 ? 1 : g);
}

bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

}  // namespace
}  // namespace mmb

extern "C" {

int mmb_muon_update_master(const mmb_master_update_seg* segs, int nseg, float alpha, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "mmb_muon_update_master: bad segment table");
  if (nseg == 0) return MMB_OK;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_muon_update_master: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int base = 0; base < nseg; base += MAX_SEG) {
    Table tab;
    tab.nseg = (nseg - base) < MAX_SEG ? (nseg - base) : MAX_SEG;
    long long vecs = 0;
    for (int i = 0; i < tab.nseg; ++i) {
      const mmb_master_update_seg& s = segs[base + i];
      MMB_REQUIRE(s.numel > 0 && s.master && s.ortho, "mmb_muon_update_master: segment %d empty", base + i);
      Seg& d = tab.seg[i];
      d.master = static_cast<float*>(s.master);
      d.shadow = static_cast<__nv_bfloat16*>(s.shadow);
      d.a = s.ortho;
      d.exp_avg = d.exp_avg_sq = nullptr;
      d.numel = s.numel;
      d.step = 0;
      d.vec_ok = aligned32(s.master) && aligned16(s.ortho) && (s.shadow == nullptr || aligned16(s.shadow));
      tab.vec_start[i] = vecs;
      vecs += (s.numel + VEC - 1) / VEC;
    }
    tab.vec_start[tab.nseg] = vecs;
    update_master_kernel<<<grid_for(vecs, sms), THREADS, 0, st>>>(tab, alpha);
    MMB_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  return MMB_OK;
}

int mmb_adamw_master_step(const mmb_master_adamw_seg* segs, int nseg, int grad_dtype, double lr, double beta1_in,
                          double beta2_in, double weight_decay, double eps_in, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "mmb_adamw_master_step: bad segment table");
  MMB_REQUIRE(grad_dtype == MMB_BF16 || grad_dtype == MMB_F32, "mmb_adamw_master_step: grad_dtype %d", grad_dtype);
  if (nseg == 0) return MMB_OK;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_adamw_master_step: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // hyper-parameters arrive as doubles, the Python floats of torch.optim, and are narrowed to fp32 here, as
  // torch's fused kernel narrows them; everything derived from them is formed in fp32 on the device
  const float lr_f = static_cast<float>(lr), wd_f = static_cast<float>(weight_decay);
  const float beta1 = static_cast<float>(beta1_in), beta2 = static_cast<float>(beta2_in), eps = static_cast<float>(eps_in);
  for (int base = 0; base < nseg; base += MAX_SEG) {
    Table tab;
    tab.nseg = (nseg - base) < MAX_SEG ? (nseg - base) : MAX_SEG;
    long long vecs = 0;
    for (int i = 0; i < tab.nseg; ++i) {
      const mmb_master_adamw_seg& s = segs[base + i];
      MMB_REQUIRE(s.numel > 0 && s.master && s.grad && s.exp_avg && s.exp_avg_sq,
                  "mmb_adamw_master_step: segment %d empty", base + i);
      MMB_REQUIRE(s.step >= 1, "mmb_adamw_master_step: segment %d has step %d (pass the incremented count)", base + i,
                  s.step);
      Seg& d = tab.seg[i];
      d.master = static_cast<float*>(s.master);
      d.shadow = static_cast<__nv_bfloat16*>(s.shadow);
      d.a = s.grad;
      d.exp_avg = static_cast<float*>(s.exp_avg);
      d.exp_avg_sq = static_cast<float*>(s.exp_avg_sq);
      d.numel = s.numel;
      d.step = s.step;
      d.vec_ok = aligned32(s.master) && aligned32(s.exp_avg) && aligned32(s.exp_avg_sq) &&
                 (grad_dtype == MMB_F32 ? aligned32(s.grad) : aligned16(s.grad)) &&
                 (s.shadow == nullptr || aligned16(s.shadow));
      tab.vec_start[i] = vecs;
      vecs += (s.numel + VEC - 1) / VEC;
    }
    tab.vec_start[tab.nseg] = vecs;
    const int grid = grid_for(vecs, sms);
    if (grad_dtype == MMB_BF16)
      adamw_master_kernel<__nv_bfloat16><<<grid, THREADS, 0, st>>>(tab, lr_f, wd_f, beta1, beta2, eps);
    else
      adamw_master_kernel<float><<<grid, THREADS, 0, st>>>(tab, lr_f, wd_f, beta1, beta2, eps);
    MMB_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  return MMB_OK;
}

}  // extern "C"
