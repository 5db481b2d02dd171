// AdamW with both moments stored as FP8 (E4M3, groups of 128), one pass.
//
// The reference's FP8-state optimizer dequantises every state tensor to fp32,
// runs the unchanged AdamW step and quantises back
// (pretrain/src/models/monarch/coat_state_muon.py:126-139 around
// monarch_muon.py:171-201): for each moment a read of the codes, an fp32 write,
// the AdamW kernels over fp32 moments, and a re-read plus a write of codes.
// Here a group of 128 elements is decoded, stepped and re-encoded in registers:
// HBM traffic per element is the parameter (in/out), the gradient and two code
// bytes in and out - 10 bytes with bf16 parameters instead of about 40.
//
// Arithmetic follows the reference's op order with fp32 moments: decoupled
// decay multiplies the parameter first (rounded to its dtype), the moments are
// updated in fp32 (the gradient is promoted), eps is added after
// sqrt(v)/sqrt(bc2), the parameter update is rounded once to its dtype.
// exp_avg is a signed state, exp_avg_sq an unsigned one (coat_state_muon.py:19).
#include <cmath>

#include "fp8_codec.cuh"

namespace mmb {
namespace {

constexpr int MAX_SEG = 64;
constexpr int THREADS = 256;
constexpr int UNIT = 4096;  // elements per warp work unit

struct Seg {
  void* param;
  const void* grad;
  uint8_t* m_codes;
  uint8_t* v_codes;
  float* m_scale; float* m_expand; float* m_sqrt;
  float* v_scale; float* v_expand; float* v_sqrt;
  long long numel;
  float inv_bc2_sqrt, step_size;   // 1 / sqrt(1 - beta2^step) formed in double (torch multiplies by the reciprocal)
  int vec_ok;
  int pad_;
};
struct Table {
  Seg seg[MAX_SEG];
  long long unit_start[MAX_SEG + 1];
  int nseg;
};

template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return bf16_round(v); }
template <>
__device__ __forceinline__ float round_to<float>(float v) { return v; }

// Decode 16 codes of one lane (already converted to float) in place.
template <int FORMAT, int DIV>
__device__ __forceinline__ void decode16(float* x, float s, float expand, float sqrt_mm, bool is_signed) {
  if (FORMAT == MMB_STATE_FP8_ABSMAX) {
#pragma unroll
    for (int i = 0; i < ELEMS_PER_LANE; ++i) x[i] = __fmul_rn(x[i], s);
    return;
  }
  const float inv_expand = fdiv<DIV>(1.0f, fmaxf(expand, 1e-30f));
  const float sq = fmaxf(sqrt_mm, 1e-30f);
  const bool hw = DIV == MMB_DIV_IEEE && inv_expand <= POW_HW_MAX_EXPONENT;  // uniform over the group
#pragma unroll
  for (int i = 0; i < ELEMS_PER_LANE; ++i) {
    float scaled = __fmul_rn(x[i], s);
    if (!is_signed) scaled = fmaxf(scaled, 0.0f);
    const float a = fabsf(scaled);
    const float pw = hw ? pow_hw(fmaxf(a, 1e-30f), inv_expand) : pow_lib(fmaxf(a, 1e-30f), inv_expand);
    x[i] = a > 0.0f ? __fmul_rn(with_sign_of(pw, scaled), sq) : 0.0f;
  }
}

// Encode 16 values of one lane (elements i >= n are padding and must be 0): group statistics over the
// 8 lanes of the group, the group's parameters, the quotients to be cast to E4M3.
template <int FORMAT, int DIV>
__device__ __forceinline__ void encode16(const float* m, float expand_min, bool is_signed, float* q, ExpandParams& ep) {
  float amax = 0.0f, amin = 3.4028235e38f;
#pragma unroll
  for (int i = 0; i < ELEMS_PER_LANE; ++i) {
    const float a = fabsf(m[i]);
    amax = fmaxf(amax, a);
    if (FORMAT == MMB_STATE_FP8_EXPAND && a > 0.0f) amin = fminf(amin, a);
  }
  amax = group_max(amax);
  if (FORMAT == MMB_STATE_FP8_ABSMAX) {
    ep.scale = fdiv<DIV>(__fadd_rn(amax, 1e-20f), 448.0f);
    ep.expand = 1.0f;
    ep.sqrt_mm = 1.0f;
    if (DIV == MMB_DIV_IEEE && markstein_ok(ep.scale)) {
      const float r = __frcp_rn(ep.scale);
#pragma unroll
      for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = quotient_markstein(m[i], ep.scale, r);
    } else {
#pragma unroll
      for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = fdiv<DIV>(m[i], ep.scale);
    }
    return;
  }
  amin = group_min(amin);
  ep = expand_group_params<DIV, DIV == MMB_DIV_IEEE>(amax, amin, amin < 3.4028235e38f, expand_min);
  const bool quick = DIV == MMB_DIV_IEEE && ep.expand <= POW_HW_MAX_EXPONENT && markstein_ok(ep.sqrt_mm) &&
                     markstein_ok(ep.scale) && amin >= 1e-30f && ep.sqrt_mm >= 1e-30f && amax <= amin * 1e30f;
  if (quick) {
    const float r_sq = __frcp_rn(ep.sqrt_mm), r_s = __frcp_rn(ep.scale);
#pragma unroll
    for (int i = 0; i < ELEMS_PER_LANE; ++i) {
      const float a = fabsf(m[i]);
      const float base = quotient_markstein(a, ep.sqrt_mm, r_sq);
      float pw = pow_hw(base, ep.expand);
      if (is_signed) pw = with_sign_of(pw, m[i]);
      q[i] = quotient_markstein(a > 0.0f ? pw : 0.0f, ep.scale, r_s);
    }
  } else {
#pragma unroll
    for (int i = 0; i < ELEMS_PER_LANE; ++i) {
      const float v = expand_normalize_general<DIV>(is_signed ? m[i] : fabsf(m[i]), ep.sqrt_mm, ep.expand, ep.scale);
      q[i] = v;
    }
  }
}

template <int FORMAT, typename T, int DIV>
__global__ void __launch_bounds__(THREADS, 2)
adamw_fp8_kernel(const __grid_constant__ Table tab, float decay, float beta1, float one_m_beta1, float beta2,
                 float one_m_beta2, float eps, float expand_min, const float* __restrict__ grad_scale_dev) {
  const float gscale = grad_scale_dev != nullptr ? *grad_scale_dev : 1.0f;
  const int lane = threadIdx.x & 31;
  const int sub = lane & (LANES_PER_GROUP - 1);
  const int grp_in_warp = lane >> 3;
  const long long warp_global = static_cast<long long>(blockIdx.x) * (THREADS / 32) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (THREADS / 32);
  const long long total_units = tab.unit_start[tab.nseg];

  for (long long u = warp_global; u < total_units; u += nwarps) {
    int lo = 0, hi = tab.nseg;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tab.unit_start[mid] <= u) lo = mid; else hi = mid;
    }
    const Seg& sg = tab.seg[lo];
    const long long e0 = (u - tab.unit_start[lo]) * UNIT;
    long long e1 = e0 + UNIT;
    if (e1 > sg.numel) e1 = sg.numel;
    const int ngroups = static_cast<int>((e1 - e0 + GROUP - 1) / GROUP);

    for (int g0 = 0; g0 < ngroups; g0 += 4) {
      const int gi = g0 + grp_in_warp;
      const bool active = gi < ngroups;
      const long long gstart = e0 + static_cast<long long>(gi) * GROUP;
      const long long at = gstart + sub * ELEMS_PER_LANE;
      int n = 0;
      if (active) {
        const long long rem = sg.numel - at;
        n = rem >= ELEMS_PER_LANE ? ELEMS_PER_LANE : (rem > 0 ? static_cast<int>(rem) : 0);
      }
      const bool vec = sg.vec_ok && n == ELEMS_PER_LANE;
      const long long gidx = gstart / GROUP;

      float p[ELEMS_PER_LANE], g[ELEMS_PER_LANE], m[ELEMS_PER_LANE], v[ELEMS_PER_LANE];
#pragma unroll
      for (int i = 0; i < ELEMS_PER_LANE; ++i) { p[i] = 0.0f; g[i] = 0.0f; m[i] = 0.0f; v[i] = 0.0f; }
      if (n > 0) {
        Elem<T>::load16(sg.param, at, vec, n, p);
        Elem<T>::load16(sg.grad, at, vec, n, g);
        load_codes16(sg.m_codes + at, vec, n, m);
        load_codes16(sg.v_codes + at, vec, n, v);
        const bool ex = FORMAT == MMB_STATE_FP8_EXPAND;
        decode16<FORMAT, DIV>(m, sg.m_scale[gidx], ex ? sg.m_expand[gidx] : 1.0f, ex ? sg.m_sqrt[gidx] : 1.0f, true);
        decode16<FORMAT, DIV>(v, sg.v_scale[gidx], ex ? sg.v_expand[gidx] : 1.0f, ex ? sg.v_sqrt[gidx] : 1.0f, false);
      }

#pragma unroll
      for (int i = 0; i < ELEMS_PER_LANE; ++i) {
        float gi_f = g[i];
        if (gscale != 1.0f) gi_f = round_to<T>(__fmul_rn(gi_f, gscale));            // like grad.mul_(coef) on the stored type
        float pi = p[i];
        if (decay != 1.0f) pi = round_to<T>(__fmul_rn(pi, decay));                   // p.mul_(1 - lr*wd)
        const float mi = fmaf(one_m_beta1, gi_f, __fmul_rn(m[i], beta1));            // exp_avg.mul_(b1).add_(g, alpha=1-b1)
        const float vi = fmaf(one_m_beta2, __fmul_rn(gi_f, gi_f), __fmul_rn(v[i], beta2));  // .mul_(b2).addcmul_(g, g, 1-b2): a + value*(b*c)
        const float d = __fadd_rn(__fmul_rn(__fsqrt_rn(vi), sg.inv_bc2_sqrt), eps);  // sqrt(v)/sqrt(bc2) + eps, the division as torch does it
        pi = round_to<T>(fmaf(-sg.step_size, __fdiv_rn(mi, d), pi));                 // p.addcdiv_(m, denom, value=-lr/bc1)
        const bool valid = i < n;
        p[i] = pi;
        m[i] = valid ? mi : 0.0f;
        v[i] = valid ? vi : 0.0f;
      }

      float q[ELEMS_PER_LANE];
      ExpandParams ep;
      encode16<FORMAT, DIV>(m, expand_min, true, q, ep);
      if (n > 0) {
        store_codes16(sg.m_codes + at, vec, n, q);
        if (sub == 0) {
          sg.m_scale[gidx] = ep.scale;
          if (FORMAT == MMB_STATE_FP8_EXPAND) { sg.m_expand[gidx] = ep.expand; sg.m_sqrt[gidx] = ep.sqrt_mm; }
        }
      }
      encode16<FORMAT, DIV>(v, expand_min, false, q, ep);
      if (n > 0) {
        store_codes16(sg.v_codes + at, vec, n, q);
        if (sub == 0) {
          sg.v_scale[gidx] = ep.scale;
          if (FORMAT == MMB_STATE_FP8_EXPAND) { sg.v_expand[gidx] = ep.expand; sg.v_sqrt[gidx] = ep.sqrt_mm; }
        }
        Elem<T>::store16(sg.param, at, vec, n, p);
      }
    }
  }
}

}  // namespace
}  // namespace mmb

extern "C" {

int mmb_adamw_fp8_step(const mmb_adamw_fp8_seg* segs, int nseg, int dtype, int state_format, int div_mode, double lr_in,
                       double beta1_in, double beta2_in, double weight_decay_in, double eps_in, int expand_min, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "mmb_adamw_fp8_step: bad segment table");
  MMB_REQUIRE(dtype == MMB_BF16 || dtype == MMB_F32, "mmb_adamw_fp8_step: dtype %d", dtype);
  MMB_REQUIRE(state_format == MMB_STATE_FP8_ABSMAX || state_format == MMB_STATE_FP8_EXPAND,
              "mmb_adamw_fp8_step: state_format %d is not an FP8 format", state_format);
  MMB_REQUIRE(div_mode >= MMB_DIV_IEEE && div_mode <= MMB_DIV_IEEE_STRICT, "mmb_adamw_fp8_step: div_mode %d", div_mode);
  MMB_REQUIRE(expand_min >= 1, "mmb_adamw_fp8_step: expand_min %d", expand_min);
  if (nseg == 0) return MMB_OK;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_adamw_fp8_step: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // doubles in, as the reference's Python floats; derived scalars formed in double, narrowed once
  const double b1 = beta1_in, b2 = beta2_in, lrd = lr_in, wd = weight_decay_in;
  const float beta1 = static_cast<float>(b1), beta2 = static_cast<float>(b2), eps = static_cast<float>(eps_in);
  const float decay = wd > 0.0 ? static_cast<float>(1.0 - lrd * wd) : 1.0f;
  const float omb1 = static_cast<float>(1.0 - b1), omb2 = static_cast<float>(1.0 - b2);
  const uintptr_t amask = dtype == MMB_F32 ? 31u : 15u;
  for (int base = 0; base < nseg; base += MAX_SEG) {
    Table tab;
    tab.nseg = (nseg - base) < MAX_SEG ? (nseg - base) : MAX_SEG;
    long long units = 0;
    for (int i = 0; i < tab.nseg; ++i) {
      const mmb_adamw_fp8_seg& s = segs[base + i];
      MMB_REQUIRE(s.numel > 0 && s.param && s.grad && s.exp_avg && s.exp_avg_sq && s.scale_exp_avg && s.scale_exp_avg_sq,
                  "mmb_adamw_fp8_step: segment %d empty", base + i);
      if (state_format == MMB_STATE_FP8_EXPAND)
        MMB_REQUIRE(s.expand_exp_avg && s.sqrt_minmax_exp_avg && s.expand_exp_avg_sq && s.sqrt_minmax_exp_avg_sq,
                    "mmb_adamw_fp8_step: segment %d lacks expand/sqrt_minmax arrays", base + i);
      MMB_REQUIRE(s.step >= 1, "mmb_adamw_fp8_step: segment %d has step %d (must be >= 1)", base + i, s.step);
      Seg& d = tab.seg[i];
      d.param = s.param;
      d.grad = s.grad;
      d.m_codes = static_cast<uint8_t*>(s.exp_avg);
      d.v_codes = static_cast<uint8_t*>(s.exp_avg_sq);
      d.m_scale = s.scale_exp_avg; d.m_expand = s.expand_exp_avg; d.m_sqrt = s.sqrt_minmax_exp_avg;
      d.v_scale = s.scale_exp_avg_sq; d.v_expand = s.expand_exp_avg_sq; d.v_sqrt = s.sqrt_minmax_exp_avg_sq;
      d.numel = s.numel;
      const double bc1 = 1.0 - std::pow(b1, static_cast<double>(s.step));
      const double bc2 = 1.0 - std::pow(b2, static_cast<double>(s.step));
      d.inv_bc2_sqrt = static_cast<float>(1.0 / std::sqrt(bc2));
      d.step_size = static_cast<float>(lrd / bc1);
      d.vec_ok = (((reinterpret_cast<uintptr_t>(s.param) | reinterpret_cast<uintptr_t>(s.grad)) & amask) == 0) &&
                 aligned16(s.exp_avg) && aligned16(s.exp_avg_sq);
      tab.unit_start[i] = units;
      units += (s.numel + UNIT - 1) / UNIT;
    }
    tab.unit_start[tab.nseg] = units;
    const long long warps_per_cta = THREADS / 32;
    long long want = (units + warps_per_cta - 1) / warps_per_cta;
    const long long cap = stream_grid_cap(sms) < static_cast<long long>(sms) * 8 ? stream_grid_cap(sms) : static_cast<long long>(sms) * 8;
    const int grid = static_cast<int>(want < cap ? (want < 1 ? 1 : want) : cap);
    const float em = static_cast<float>(expand_min);
#define MMB_LAUNCH(F, T, D) \
  adamw_fp8_kernel<F, T, D><<<grid, THREADS, 0, st>>>(tab, decay, beta1, omb1, beta2, omb2, eps, em, device_grad_scale())
#define MMB_LAUNCH_DIV(F, T)                                                   \
  do {                                                                         \
    if (div_mode == MMB_DIV_IEEE) MMB_LAUNCH(F, T, MMB_DIV_IEEE);              \
    else if (div_mode == MMB_DIV_FULL) MMB_LAUNCH(F, T, MMB_DIV_FULL);         \
    else MMB_LAUNCH(F, T, MMB_DIV_IEEE_STRICT);                                \
  } while (0)
    if (state_format == MMB_STATE_FP8_ABSMAX) {
      if (dtype == MMB_BF16) MMB_LAUNCH_DIV(MMB_STATE_FP8_ABSMAX, __nv_bfloat16); else MMB_LAUNCH_DIV(MMB_STATE_FP8_ABSMAX, float);
    } else {
      if (dtype == MMB_BF16) MMB_LAUNCH_DIV(MMB_STATE_FP8_EXPAND, __nv_bfloat16); else MMB_LAUNCH_DIV(MMB_STATE_FP8_EXPAND, float);
    }
#undef MMB_LAUNCH_DIV
#undef MMB_LAUNCH
    MMB_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  return MMB_OK;
}

}  // extern "C"
