// Device-side pieces of the FP8 optimizer-state codecs, shared by the fused
// momentum kernel and the fused FP8 AdamW kernel: IEEE / approximate division,
// E4M3 conversions, the per-group statistics of COAT's range expansion
// (pretrain/src/models/monarch/coat_state_muon.py:22-91), 16-element loaders,
// and the exact three-instruction quotient.  Everything has internal linkage.
#pragma once

#include "common.cuh"

namespace mmb {
namespace {

constexpr int GROUP = 128;          // elements per quantisation group
constexpr int LANES_PER_GROUP = 8;  // a group is handled by 8 lanes x 16 elements
constexpr int ELEMS_PER_LANE = 16;

// ---------------------------------------------------------------- arithmetic
template <int DIV>
__device__ __forceinline__ float fdiv(float a, float b) {
  if (DIV != MMB_DIV_FULL) return __fdiv_rn(a, b);
  float r;
  asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// div.full.f32(a, b) is fmul.rn(a, rcp.approx.f32(b)): the two agree in every bit on 2^32 random pairs with
// |a| <= 450 |b| and b over the whole normal range (measured on a B200; the parity tests against the
// reference's kernels hold the fused kernel to that).  With a divisor shared by a whole group the reciprocal
// is formed once and each element costs one multiply.
__device__ __forceinline__ float rcp_approx(float b) {
  float r;
  asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(b));
  return r;
}
__device__ __forceinline__ bool finite_normal(float s) {
  const uint32_t e = __float_as_uint(s) & 0x7F800000u;
  return e != 0u && e != 0x7F800000u;
}

// Two fp32 operations per instruction (mul.rn.f32x2 / fma.rn.f32x2, sm_100): each half is the IEEE
// round-to-nearest result of the scalar instruction (checked bit for bit on 2^28 random triples on a B200),
// so pairing changes the instruction count, not the values.  One caution, measured: a packed add that
// consumes a packed product (and nothing else does) is contracted by the assembler into a fused
// multiply-add, .rn modifiers notwithstanding - so sums that must round separately are written with the
// scalar __fadd_rn, and add2 is only for sums whose inputs are not products.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  unsigned long long z;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(z) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&z);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  unsigned long long z;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(z) : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&z);
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  unsigned long long z;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(z)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&z);
}

template <int DIV>
__device__ __forceinline__ float fsqrt(float a) {
  if (DIV != MMB_DIV_FULL) return __fsqrt_rn(a);
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}

__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t pair) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(pair), __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

__device__ __forceinline__ uint16_t float2_to_e4m3x2(float lo, float hi) {
  return static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// pow(x, y) for normal x > 0 through the special-function unit: 2^(y*log2 x) with lg2.approx and
// ex2.approx (absolute error of the logarithm about 2^-22.6, relative error of the exponential about
// 2^-22), the product's rounding error carried into the result.  For |y| <= 4 the result is within about
// 1e-6 of the true power, which moves an E4M3 code (relative spacing 2^-3) in roughly one element out of
// 10^5.  Callers use it only in that range; larger exponents take the library powf.
__device__ __forceinline__ float pow_hw(float x, float y) {
  float l, r;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(x));
  const float th = __fmul_rn(l, y);
  const float tl = __fmaf_rn(l, y, -th);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(th));
  return __fmaf_rn(r, __fmul_rn(tl, 0.6931471806f), r);
}
__device__ __noinline__ float pow_lib(float x, float y) { return powf(x, y); }
// magnitude (>= 0) with the sign bit of s: one logic instruction.  The callers replace the result by 0
// when s is +-0, so the sign given to a zero does not matter.
__device__ __forceinline__ float with_sign_of(float magnitude, float s) {
  return __uint_as_float(__float_as_uint(magnitude) | (__float_as_uint(s) & 0x80000000u));
}
constexpr float POW_HW_MAX_EXPONENT = 4.0f;

__device__ __forceinline__ float group_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}
__device__ __forceinline__ float group_min(float v) {
  v = fminf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fminf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fminf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}
__device__ __forceinline__ int group_or(int v) {
  v |= __shfl_xor_sync(0xffffffffu, v, 1);
  v |= __shfl_xor_sync(0xffffffffu, v, 2);
  v |= __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

// COAT dynamic-range expansion, per group (pretrain/src/models/monarch/
// coat_state_muon.py:56-86).  Inputs are the group's reduced statistics.
struct ExpandParams {
  float scale, expand, sqrt_mm;
};

template <int DIV, bool HW_POW = false>
__device__ __forceinline__ ExpandParams expand_group_params(float absmax, float absmin_nz, bool any_nz,
                                                            float expand_min) {
  const float eps = 1e-30f;
  absmax = fmaxf(absmax, eps);
  float absmin = any_nz ? fmaxf(absmin_nz, eps) : eps;
  const float one_eps = 1.0f + eps;  // == 1.0f
  float ratio = fmaxf(fdiv<DIV>(absmax, absmin), one_eps);
  const float ratio_upper = 448.0f * 448.0f / 2.0f;
  float log_ratio = log2f(ratio);
  float safe_log = log_ratio > eps ? log_ratio : 1.0f;
  float raw = fdiv<DIV>(floorf(fdiv<DIV>(log2f(ratio_upper), safe_log) * expand_min), expand_min);
  float min_expand = fdiv<DIV>(1.0f, expand_min);
  ExpandParams p;
  p.expand = (ratio <= one_eps) ? 1.0f : fmaxf(raw, min_expand);
  p.sqrt_mm = fmaxf(fsqrt<DIV>(absmax) * fsqrt<DIV>(absmin), eps);
  float scale_base = fmaxf(fdiv<DIV>(absmax, p.sqrt_mm), eps);
  const float pw = (HW_POW && p.expand <= POW_HW_MAX_EXPONENT) ? pow_hw(scale_base, p.expand) : powf(scale_base, p.expand);
  p.scale = fmaxf(fdiv<DIV>(pw, 448.0f), eps);
  return p;
}

template <int DIV>
__device__ __forceinline__ float expand_normalize(float m, bool valid, const ExpandParams& p, bool is_signed) {
  const float eps = 1e-30f;
  float a = fabsf(m);
  float base = fmaxf(fdiv<DIV>(a, p.sqrt_mm), eps);
  float pw = powf(base, p.expand);
  float sgn = (m >= 0.0f) ? 1.0f : -1.0f;
  float n = (valid && a > 0.0f) ? (is_signed ? sgn * pw : pw) : 0.0f;
  return fdiv<DIV>(n, p.scale);
}

// Out-of-line twin of expand_normalize for the fused kernel's rare groups (huge exponent, a scale whose
// reciprocal cannot be corrected exactly, denormal inputs).
template <int DIV>
__device__ __noinline__ float expand_normalize_general(float m, float sqrt_mm, float expand, float scale) {
  ExpandParams p;
  p.scale = scale; p.expand = expand; p.sqrt_mm = sqrt_mm;
  return expand_normalize<DIV>(m, true, p, true);
}

template <int DIV>
__device__ __forceinline__ float expand_decode(float raw, float s, float expand, float sqrt_mm, bool is_signed) {
  const float eps = 1e-30f;
  expand = fmaxf(expand, eps);
  sqrt_mm = fmaxf(sqrt_mm, eps);
  float scaled = raw * s;
  if (!is_signed) scaled = fmaxf(scaled, 0.0f);
  float a = fabsf(scaled);
  float sgn = (scaled >= 0.0f) ? 1.0f : -1.0f;
  float pw = powf(fmaxf(a, eps), fdiv<DIV>(1.0f, expand));
  return a > 0.0f ? sgn * pw * sqrt_mm : 0.0f;
}

// ------------------------------------------------------------------- loaders
template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ void load16(const void* base, long long at, bool vec, int n, float* out) {
    const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(base) + at;
    if (vec) {
      uint4 v[2];
      v[0] = __ldcs(reinterpret_cast<const uint4*>(p));
      v[1] = __ldcs(reinterpret_cast<const uint4*>(p) + 1);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x;
        out[2 * i + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) out[i] = i < n ? __bfloat162float(p[i]) : 0.0f;
    }
  }
  static __device__ __forceinline__ void store16(void* base, long long at, bool vec, int n, const float* in) {
    __nv_bfloat16* p = static_cast<__nv_bfloat16*>(base) + at;
    if (vec) {
      uint4 v[2];
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
      reinterpret_cast<uint4*>(p)[0] = v[0];
      reinterpret_cast<uint4*>(p)[1] = v[1];
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (i < n) p[i] = __float2bfloat16_rn(in[i]);
    }
  }
};
template <>
struct Elem<float> {
  static __device__ __forceinline__ void load16(const void* base, long long at, bool vec, int n, float* out) {
    const float* p = static_cast<const float*>(base) + at;
    if (vec) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float4 f = __ldcs(reinterpret_cast<const float4*>(p) + i);
        out[4 * i] = f.x;
        out[4 * i + 1] = f.y;
        out[4 * i + 2] = f.z;
        out[4 * i + 3] = f.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) out[i] = i < n ? p[i] : 0.0f;
    }
  }
  static __device__ __forceinline__ void store16(void* base, long long at, bool vec, int n, const float* in) {
    float* p = static_cast<float*>(base) + at;
    if (vec) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        reinterpret_cast<float4*>(p)[i] = make_float4(in[4 * i], in[4 * i + 1], in[4 * i + 2], in[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (i < n) p[i] = in[i];
    }
  }
};

__device__ __forceinline__ void load_codes16(const uint8_t* p, bool vec, int n, float* out) {
  if (vec) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint16_t* h = reinterpret_cast<const uint16_t*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float2 f = e4m3x2_to_float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = i < n ? e4m3x2_to_float2(p[i]).x : 0.0f;
  }
}

__device__ __forceinline__ void store_codes16(uint8_t* p, bool vec, int n, const float* q) {
  if (vec) {
    uint4 v;
    uint16_t* h = reinterpret_cast<uint16_t*>(&v);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = float2_to_e4m3x2(q[2 * i], q[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = v;
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i < n) p[i] = static_cast<uint8_t>(float2_to_e4m3x2(q[i], 0.0f) & 0xff);
  }
}

// m / s rounded like IEEE division in three instructions.  With r = rn(1/s) and
// q0 = rn(m*r), the residual e = m - q0*s is exact in one fused multiply-add and
// rn(q0 + e*r) is the correctly rounded quotient (Markstein's correction step,
// the core of the compiler's own division), provided s is finite, its mantissa
// is not all ones and nothing underflows.  The caller checks s once per group
// (`markstein_ok`); an element so small that the residual could underflow has a
// quotient below 2^-27, far under half of E4M3's smallest subnormal, and is
// encoded as a signed zero by any approximation.
__device__ __forceinline__ bool markstein_ok(float s) {
  const uint32_t b = __float_as_uint(s);
  return (b & 0x7F800000u) != 0x7F800000u && (b & 0x007FFFFFu) != 0x007FFFFFu;
}
__device__ __forceinline__ float quotient_markstein(float m, float s, float r) {
  const float q0 = __fmul_rn(m, r);
  const float e = __fmaf_rn(-q0, s, m);
  return __fmaf_rn(e, r, q0);
}

}  // namespace
}  // namespace mmb
