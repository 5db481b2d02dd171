// Heavy-ball momentum fused with the optimizer-state codec.
//
// One streaming pass per step: read the stored state (E4M3 codes + per-group
// fp32 scale, or a plain bf16/fp32 buffer) and the gradient, form
// m = round(beta*m) then m = round(m + g) - two roundings, like the
// reference's mul_ followed by add_ (pretrain/src/models/monarch/
// monarch_muon.py:148) - requantise, and emit what Newton-Schulz needs: the
// bf16 copy of m and per-block sums of squares of m.
//
// Work decomposition.  A group is 128 contiguous elements and is handled by 8
// lanes x 16 elements, so the group maximum is three xor-shuffles and every
// global access is a 16-byte vector.  A warp walks a "unit" of 4096 elements
// of one block and leaves one partial sum of squares; a second tiny kernel
// adds a block's partials in a fixed order, which keeps the norm - and so the
// whole step - bit-reproducible from run to run (no float atomics).
//
// HBM traffic per element with the absmax codec and bf16 gradients:
// 1 (code in) + 2 (grad) + 1 (code out) + 2 (bf16 m) + 8/128 (scale in/out)
// = 6.0625 bytes; the kernel is bandwidth bound.
#include "fp8_codec.cuh"

#include <atomic>

namespace mmb {
namespace {

constexpr int UNIT = 4096;  // elements per warp work unit = one partial sum
constexpr int MAX_SEG = 96;
constexpr int THREADS = 256;

struct SegDev {
  const void* grad;
  void* state;
  float* scale;
  float* expand;
  float* sqrt_mm;
  __nv_bfloat16* m_out;
  long long numel;
  long long block_elems;   // multiple of 128, or == numel
  long long partial_base;  // first partial of this segment in the scratch
  long long first_block;
  int cpb;                 // units (= partials) per block
  int vec_ok;              // all pointers 16-byte aligned
};

struct SegTable {
  SegDev seg[MAX_SEG];
  long long unit_start[MAX_SEG + 1];
  long long block_start[MAX_SEG + 1];  // launch-wide numbering of blocks
  int nseg;
};

// ------------------------------------------------- fast path (FP8 absmax, full groups)
// Raw 16-byte loads of one lane's share of a group, kept undecoded so that the
// next group's loads can be in flight while the current one is computed.
template <typename GradT>
struct RawGroup {
  uint4 codes;
  uint4 grad[sizeof(GradT) == 2 ? 2 : 4];
  float scale;
  float expand, sqrt_mm;  // range-expansion codec only
};

template <int FORMAT, typename GradT>
__device__ __forceinline__ void load_raw(RawGroup<GradT>& r, const SegDev& sg, long long at) {
  r.codes = __ldcs(reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(sg.state) + at));
  const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const GradT*>(sg.grad) + at);
#pragma unroll
  for (int i = 0; i < (sizeof(GradT) == 2 ? 2 : 4); ++i) r.grad[i] = __ldcs(gp + i);
  r.scale = __ldg(sg.scale + at / GROUP);
  if (FORMAT == MMB_STATE_FP8_EXPAND) {
    r.expand = __ldg(sg.expand + at / GROUP);
    r.sqrt_mm = __ldg(sg.sqrt_mm + at / GROUP);
  }
}

template <typename GradT>
__device__ __forceinline__ float raw_grad(const RawGroup<GradT>& r, int i) {
  if (sizeof(GradT) == 2) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(r.grad)[i >> 1];
    return __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));  // bf16 -> fp32 is a shift
  }
  return reinterpret_cast<const float*>(r.grad)[i];
}

// Plain bf16 state (the reference's own format with bf16 parameters), aligned pointers, full groups: the
// same two-groups-in-flight pipeline without a codec.  m = bf16(beta*m), m = bf16(m + g): the two
// roundings of mul_ followed by add_ on a bf16 tensor.  Returns this lane's share of sum(m^2).
template <typename GradT>
__device__ __forceinline__ float bf16_state_unit(const SegDev& sg, long long e0, int ngroups, int grp_in_warp, int sub,
                                                 float beta, float grad_scale) {
  struct Raw {
    uint4 st[2];
    uint4 grad[sizeof(GradT) == 2 ? 2 : 4];
  };
  auto load = [&](Raw& r, long long at) {
    const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(sg.state) + at);
    r.st[0] = __ldcs(sp);
    r.st[1] = __ldcs(sp + 1);
    const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const GradT*>(sg.grad) + at);
#pragma unroll
    for (int i = 0; i < (sizeof(GradT) == 2 ? 2 : 4); ++i) r.grad[i] = __ldcs(gp + i);
  };
  const bool scaled = grad_scale != 1.0f;
  const bool separate_out = sg.m_out != nullptr && static_cast<void*>(sg.m_out) != sg.state;
  float ss = 0.0f;
  Raw cur, nxt;
  bool cur_ok = grp_in_warp < ngroups;
  if (cur_ok) load(cur, e0 + static_cast<long long>(grp_in_warp) * GROUP + sub * ELEMS_PER_LANE);
  for (int g0 = 0; g0 < ngroups; g0 += 4) {
    const int gi_next = g0 + 4 + grp_in_warp;
    const bool nxt_ok = gi_next < ngroups;
    if (nxt_ok) load(nxt, e0 + static_cast<long long>(gi_next) * GROUP + sub * ELEMS_PER_LANE);
    if (cur_ok) {
      const long long at = e0 + static_cast<long long>(g0 + grp_in_warp) * GROUP + sub * ELEMS_PER_LANE;
      uint4 mv[2];
      __nv_bfloat162* mh = reinterpret_cast<__nv_bfloat162*>(mv);
      const uint32_t* sw = reinterpret_cast<const uint32_t*>(cur.st);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float g[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int e = 2 * i + j;
          if (sizeof(GradT) == 2) {
            const uint32_t w = reinterpret_cast<const uint32_t*>(cur.grad)[e >> 1];
            g[j] = __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
          } else {
            g[j] = reinterpret_cast<const float*>(cur.grad)[e];
          }
          if (scaled) {
            g[j] = __fmul_rn(g[j], grad_scale);
            if (sizeof(GradT) == 2) g[j] = bf16_round(g[j]);
          }
        }
        // both roundings as packed conversions of the pair; the second one is also what gets stored
        const float m0 = __uint_as_float(sw[i] << 16), m1 = __uint_as_float(sw[i] & 0xffff0000u);
        const float2 x = __bfloat1622float2(__floats2bfloat162_rn(__fmul_rn(beta, m0), __fmul_rn(beta, m1)));
        mh[i] = __floats2bfloat162_rn(__fadd_rn(x.x, g[0]), __fadd_rn(x.y, g[1]));
        const float2 y = __bfloat1622float2(mh[i]);
        ss = fmaf(y.x, y.x, ss);
        ss = fmaf(y.y, y.y, ss);
      }
      uint4* sp = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(sg.state) + at);
      sp[0] = mv[0];
      sp[1] = mv[1];
      if (separate_out) {
        uint4* mp = reinterpret_cast<uint4*>(sg.m_out + at);
        mp[0] = mv[0];
        mp[1] = mv[1];
      }
    }
    cur = nxt;
    cur_ok = nxt_ok;
  }
  return ss;
}

// Plain fp32 state (the reference's pretraining recipe: fp32 parameters and momentum), same pipeline:
// m = rn(beta*m), m = rn(m + g) in fp32, bf16 copy for Newton-Schulz, sum of squares of the fp32 values.
template <typename GradT>
__device__ __forceinline__ float f32_state_unit(const SegDev& sg, long long e0, int ngroups, int grp_in_warp, int sub,
                                                float beta, float grad_scale) {
  struct Raw {
    uint4 st[4];
    uint4 grad[sizeof(GradT) == 2 ? 2 : 4];
  };
  auto load = [&](Raw& r, long long at) {
    const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const float*>(sg.state) + at);
#pragma unroll
    for (int i = 0; i < 4; ++i) r.st[i] = __ldcs(sp + i);
    const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const GradT*>(sg.grad) + at);
#pragma unroll
    for (int i = 0; i < (sizeof(GradT) == 2 ? 2 : 4); ++i) r.grad[i] = __ldcs(gp + i);
  };
  const bool scaled = grad_scale != 1.0f;
  float ss = 0.0f;
  Raw cur, nxt;
  bool cur_ok = grp_in_warp < ngroups;
  if (cur_ok) load(cur, e0 + static_cast<long long>(grp_in_warp) * GROUP + sub * ELEMS_PER_LANE);
  for (int g0 = 0; g0 < ngroups; g0 += 4) {
    const int gi_next = g0 + 4 + grp_in_warp;
    const bool nxt_ok = gi_next < ngroups;
    if (nxt_ok) load(nxt, e0 + static_cast<long long>(gi_next) * GROUP + sub * ELEMS_PER_LANE);
    if (cur_ok) {
      const long long at = e0 + static_cast<long long>(g0 + grp_in_warp) * GROUP + sub * ELEMS_PER_LANE;
      uint4 sv[4], mv[2];
      float* sf = reinterpret_cast<float*>(sv);
      __nv_bfloat162* mh = reinterpret_cast<__nv_bfloat162*>(mv);
      const float* old = reinterpret_cast<const float*>(cur.st);
#pragma unroll
      for (int e = 0; e < ELEMS_PER_LANE; ++e) {
        float g;
        if (sizeof(GradT) == 2) {
          const uint32_t w = reinterpret_cast<const uint32_t*>(cur.grad)[e >> 1];
          g = __uint_as_float((e & 1) ? (w & 0xffff0000u) : (w << 16));
        } else {
          g = reinterpret_cast<const float*>(cur.grad)[e];
        }
        if (scaled) {
          g = __fmul_rn(g, grad_scale);
          if (sizeof(GradT) == 2) g = bf16_round(g);
        }
        const float x = __fadd_rn(__fmul_rn(beta, old[e]), g);
        sf[e] = x;
        ss = fmaf(x, x, ss);
      }
      uint4* sp = reinterpret_cast<uint4*>(static_cast<float*>(sg.state) + at);
#pragma unroll
      for (int i = 0; i < 4; ++i) sp[i] = sv[i];
      if (sg.m_out != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) mh[i] = __floats2bfloat162_rn(sf[2 * i], sf[2 * i + 1]);
        uint4* mp = reinterpret_cast<uint4*>(sg.m_out + at);
        mp[0] = mv[0];
        mp[1] = mv[1];
      }
    }
    cur = nxt;
    cur_ok = nxt_ok;
  }
  return ss;
}

// FP8 absmax state, aligned pointers, full groups: the path the full-size step runs.  Two groups of loads in flight per
// lane; the arithmetic works on pairs of elements with the packed fp32 instructions (same bits as the
// scalar ones, half the issue slots).  m = rn(beta * rn(code * scale)) + g, quantised with
// scale' = (absmax + 1e-20) / 448 and code' = cvt.rn.satfinite.e4m3(m / scale').  Returns this lane's
// share of sum(m^2).
template <typename GradT, int DIV>
__device__ __forceinline__ float fp8_absmax_unit(const SegDev& sg, long long e0, int ngroups, int grp_in_warp, int sub,
                                                 float beta, float grad_scale) {
  const bool scaled = grad_scale != 1.0f;
  const float2 beta2 = make_float2(beta, beta), gs2 = make_float2(grad_scale, grad_scale);
  float2 ss2 = make_float2(0.0f, 0.0f);
  RawGroup<GradT> cur, nxt;
  bool cur_ok = grp_in_warp < ngroups;
  if (cur_ok) load_raw<MMB_STATE_FP8_ABSMAX, GradT>(cur, sg, e0 + static_cast<long long>(grp_in_warp) * GROUP + sub * ELEMS_PER_LANE);
  for (int g0 = 0; g0 < ngroups; g0 += 4) {
    const int gi_next = g0 + 4 + grp_in_warp;
    const bool nxt_ok = gi_next < ngroups;
    if (nxt_ok) load_raw<MMB_STATE_FP8_ABSMAX, GradT>(nxt, sg, e0 + static_cast<long long>(gi_next) * GROUP + sub * ELEMS_PER_LANE);
    const long long at = e0 + static_cast<long long>(g0 + grp_in_warp) * GROUP + sub * ELEMS_PER_LANE;
    float2 m[ELEMS_PER_LANE / 2];
    float amax = 0.0f;
    if (cur_ok) {
      const uint16_t* h = reinterpret_cast<const uint16_t*>(&cur.codes);
      const float2 sc2 = make_float2(cur.scale, cur.scale);
#pragma unroll
      for (int p = 0; p < ELEMS_PER_LANE / 2; ++p) {
        float2 g;
        if (sizeof(GradT) == 2) {
          const uint32_t w = reinterpret_cast<const uint32_t*>(cur.grad)[p];
          g = make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));   // bf16 -> fp32 is a shift
        } else {
          g = reinterpret_cast<const float2*>(cur.grad)[p];
        }
        if (scaled) {  // like grad.mul_(scale) on the stored gradient: rounded to the gradient's type
          g = mul2(g, gs2);
          if (sizeof(GradT) == 2) g = __bfloat1622float2(__floats2bfloat162_rn(g.x, g.y));
        }
        const float2 dec = mul2(e4m3x2_to_float2(h[p]), sc2);
        const float2 bm = mul2(beta2, dec);
        // The sum stays two scalar add.rn: the assembler was seen to contract a packed multiply followed by a
        // packed add into one fused multiply-add, which would drop the reference's second rounding
        // (buf.mul_(beta) then buf.add_(grad)); scalar add.rn is never contracted.
        const float2 t = make_float2(__fadd_rn(bm.x, g.x), __fadd_rn(bm.y, g.y));
        m[p] = t;
        amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
      }
    } else {
#pragma unroll
      for (int p = 0; p < ELEMS_PER_LANE / 2; ++p) m[p] = make_float2(0.0f, 0.0f);
    }
    amax = group_max(amax);
    const float s_new = fdiv<DIV>(__fadd_rn(amax, 1e-20f), 448.0f);
    if (cur_ok) {
      uint4 cv;
      uint16_t* ch = reinterpret_cast<uint16_t*>(&cv);
      if (DIV == MMB_DIV_IEEE && markstein_ok(s_new)) {   // uniform over the group
        const float r = __frcp_rn(s_new);
#pragma unroll
        for (int p = 0; p < ELEMS_PER_LANE / 2; ++p)
          ch[p] = float2_to_e4m3x2(quotient_markstein(m[p].x, s_new, r), quotient_markstein(m[p].y, s_new, r));
      } else if (DIV == MMB_DIV_FULL && finite_normal(s_new)) {  // uniform over the group
        const float r = rcp_approx(s_new);                        // div.full.f32(m, s) == m * rcp.approx(s)
        const float2 r2 = make_float2(r, r);
#pragma unroll
        for (int p = 0; p < ELEMS_PER_LANE / 2; ++p) {
          const float2 q = mul2(m[p], r2);
          ch[p] = float2_to_e4m3x2(q.x, q.y);
        }
      } else {
#pragma unroll
        for (int p = 0; p < ELEMS_PER_LANE / 2; ++p)
          ch[p] = float2_to_e4m3x2(fdiv<DIV>(m[p].x, s_new), fdiv<DIV>(m[p].y, s_new));
      }
      *reinterpret_cast<uint4*>(static_cast<uint8_t*>(sg.state) + at) = cv;
      if (sub == 0) sg.scale[at / GROUP] = s_new;
#pragma unroll
      for (int p = 0; p < ELEMS_PER_LANE / 2; ++p) ss2 = fma2(m[p], m[p], ss2);
      if (sg.m_out != nullptr) {
        uint4 mv[2];
        __nv_bfloat162* mh = reinterpret_cast<__nv_bfloat162*>(mv);
#pragma unroll
        for (int p = 0; p < ELEMS_PER_LANE / 2; ++p) mh[p] = __floats2bfloat162_rn(m[p].x, m[p].y);
        uint4* mp = reinterpret_cast<uint4*>(sg.m_out + at);
        mp[0] = mv[0];
        mp[1] = mv[1];
      }
    }
    cur = nxt;
    cur_ok = nxt_ok;
  }
  return ss2.x + ss2.y;
}

// -------------------------------------------------------------- fused kernel
// ALL_FAST: the host has checked that every unit of the launch qualifies for the
// fast path, so the general path is compiled out (fewer registers, more warps).
template <int FORMAT, typename GradT, int DIV, bool ALL_FAST>
// resident CTAs per SM asked of the compiler: 4 (64 registers) for the absmax fast path, 3 (80) for the
// range-expansion fast path, which carries more live values per group
__global__ void __launch_bounds__(THREADS, ALL_FAST ? ((FORMAT == MMB_STATE_FP8_ABSMAX || FORMAT == MMB_STATE_BF16) ? 4 : 3) : 1)
momentum_kernel(const __grid_constant__ SegTable tab, float beta, float grad_scale, float expand_min,
                float* __restrict__ partials, const float* __restrict__ grad_scale_dev) {
  if (grad_scale_dev != nullptr) grad_scale = __fmul_rn(grad_scale, *grad_scale_dev);  // e.g. a clip coefficient
  const int lane = threadIdx.x & 31;
  const int sub = lane & (LANES_PER_GROUP - 1);
  const int grp_in_warp = lane >> 3;
  const long long warp_global = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long total_units = tab.unit_start[tab.nseg];

  for (long long u = warp_global; u < total_units; u += nwarps) {
    int lo = 0, hi = tab.nseg;  // last segment with unit_start <= u
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (tab.unit_start[mid] <= u) lo = mid; else hi = mid;
    }
    const SegDev& sg = tab.seg[lo];
    const long long local = u - tab.unit_start[lo];
    const long long blk = local / sg.cpb;
    const int chunk = static_cast<int>(local - blk * sg.cpb);
    const long long e0 = blk * sg.block_elems + static_cast<long long>(chunk) * UNIT;
    long long e1 = e0 + UNIT;
    const long long blk_end = (blk + 1) * sg.block_elems;
    if (e1 > blk_end) e1 = blk_end;
    if (e1 > sg.numel) e1 = sg.numel;
    const int ngroups = static_cast<int>((e1 - e0 + GROUP - 1) / GROUP);
    float ss = 0.0f;

    // Fast path: FP8 absmax state, aligned pointers, only full groups.  One group of loads is kept in
    // flight ahead of the arithmetic.
    const bool fast = ALL_FAST || (sg.vec_ok && ((e1 - e0) % GROUP) == 0);
    if (FORMAT == MMB_STATE_BF16 && fast) {
      ss = bf16_state_unit<GradT>(sg, e0, ngroups, grp_in_warp, sub, beta, grad_scale);
    } else if (FORMAT == MMB_STATE_F32 && fast) {
      ss = f32_state_unit<GradT>(sg, e0, ngroups, grp_in_warp, sub, beta, grad_scale);
    } else if (FORMAT == MMB_STATE_FP8_ABSMAX && fast) {
      ss = fp8_absmax_unit<GradT, DIV>(sg, e0, ngroups, grp_in_warp, sub, beta, grad_scale);
    } else if (fast) {
      RawGroup<GradT> cur, nxt;
      bool cur_ok = grp_in_warp < ngroups;
      if (cur_ok) load_raw<FORMAT, GradT>(cur, sg, e0 + static_cast<long long>(grp_in_warp) * GROUP + sub * ELEMS_PER_LANE);
      for (int g0 = 0; g0 < ngroups; g0 += 4) {
        const int gi_next = g0 + 4 + grp_in_warp;
        const bool nxt_ok = gi_next < ngroups;
        if (nxt_ok) load_raw<FORMAT, GradT>(nxt, sg, e0 + static_cast<long long>(gi_next) * GROUP + sub * ELEMS_PER_LANE);
        const long long at = e0 + static_cast<long long>(g0 + grp_in_warp) * GROUP + sub * ELEMS_PER_LANE;
        float m[ELEMS_PER_LANE];
        float amax = 0.0f, amin = 3.4028235e38f;
        if (cur_ok) {
          const uint16_t* h = reinterpret_cast<const uint16_t*>(&cur.codes);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float2 f = e4m3x2_to_float2(h[i]);
            m[2 * i] = f.x;
            m[2 * i + 1] = f.y;
          }
          const bool scaled = grad_scale != 1.0f;
          float inv_expand = 1.0f, sq_old = 1.0f;
          if (FORMAT == MMB_STATE_FP8_EXPAND) {  // the clamps of expand_decode, once per group
            inv_expand = fdiv<DIV>(1.0f, fmaxf(cur.expand, 1e-30f));
            sq_old = fmaxf(cur.sqrt_mm, 1e-30f);
          }
          const bool dec_hw = DIV == MMB_DIV_IEEE && inv_expand <= POW_HW_MAX_EXPONENT;  // uniform over the group
#pragma unroll
          for (int i = 0; i < ELEMS_PER_LANE; ++i) {
            float g = raw_grad<GradT>(cur, i);
            if (scaled) {  // like grad.mul_(scale) on the stored gradient: rounded to the gradient's type
              g = __fmul_rn(g, grad_scale);
              if (sizeof(GradT) == 2) g = bf16_round(g);
            }
            float dec = __fmul_rn(m[i], cur.scale);
            if (FORMAT == MMB_STATE_FP8_EXPAND) {  // expand_decode(raw, s, expand, sqrt_mm, signed)
              const float a = fabsf(dec);
              const float pw = dec_hw ? pow_hw(fmaxf(a, 1e-30f), inv_expand) : pow_lib(fmaxf(a, 1e-30f), inv_expand);
              dec = a > 0.0f ? __fmul_rn(with_sign_of(pw, dec), sq_old) : 0.0f;
            }
            float t = __fmul_rn(beta, dec);
            t = __fadd_rn(t, g);
            m[i] = t;
            const float a = fabsf(t);
            amax = fmaxf(amax, a);
            if (FORMAT == MMB_STATE_FP8_EXPAND && a > 0.0f) amin = fminf(amin, a);
          }
        } else {
#pragma unroll
          for (int i = 0; i < ELEMS_PER_LANE; ++i) m[i] = 0.0f;
        }
        amax = group_max(amax);
        float s_new;
        ExpandParams ep;
        if (FORMAT == MMB_STATE_FP8_EXPAND) {
          amin = group_min(amin);
          ep = expand_group_params<DIV, DIV == MMB_DIV_IEEE>(amax, amin, amin < 3.4028235e38f, expand_min);
          s_new = ep.scale;
        } else {
          s_new = fdiv<DIV>(__fadd_rn(amax, 1e-20f), 448.0f);
        }
        if (cur_ok) {
          float q[ELEMS_PER_LANE];
          if (FORMAT == MMB_STATE_FP8_EXPAND) {
            // expand_normalize per element.  Both divisions are by group constants; when the group's
            // numbers allow it (uniform over the group) they are formed exactly from a reciprocal, and
            // the power goes through the special-function unit; otherwise the general helpers run.
            const bool quick = DIV == MMB_DIV_IEEE && ep.expand <= POW_HW_MAX_EXPONENT && markstein_ok(ep.sqrt_mm) &&
                               markstein_ok(s_new) && amin >= 1e-30f && ep.sqrt_mm >= 1e-30f && amax <= amin * 1e30f;
            if (quick) {
              const float r_sq = __frcp_rn(ep.sqrt_mm), r_s = __frcp_rn(s_new);
#pragma unroll
              for (int i = 0; i < ELEMS_PER_LANE; ++i) {
                const float a = fabsf(m[i]);
                // absmax/absmin <= 1e30 (checked in `quick`) keeps the quotient of a non-zero element above
                // 1e-15, so the reference's clamp at 1e-30 never acts; a == 0 yields a NaN power that the
                // select below discards
                const float base = quotient_markstein(a, ep.sqrt_mm, r_sq);
                const float pw = with_sign_of(pow_hw(base, ep.expand), m[i]);
                q[i] = quotient_markstein(a > 0.0f ? pw : 0.0f, s_new, r_s);
              }
            } else {
#pragma unroll
              for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = expand_normalize_general<DIV>(m[i], ep.sqrt_mm, ep.expand, s_new);
            }
          } else if (DIV == MMB_DIV_IEEE && markstein_ok(s_new)) {   // uniform over the group
            const float r = __frcp_rn(s_new);
#pragma unroll
            for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = quotient_markstein(m[i], s_new, r);
          } else if (DIV == MMB_DIV_FULL && finite_normal(s_new)) {  // uniform over the group
            const float r = rcp_approx(s_new);                        // div.full.f32(m, s) == m * rcp.approx(s)
#pragma unroll
            for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = __fmul_rn(m[i], r);
          } else {
#pragma unroll
            for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = fdiv<DIV>(m[i], s_new);
          }
          uint4 cv;
          uint16_t* ch = reinterpret_cast<uint16_t*>(&cv);
#pragma unroll
          for (int i = 0; i < 8; ++i) ch[i] = float2_to_e4m3x2(q[2 * i], q[2 * i + 1]);
          *reinterpret_cast<uint4*>(static_cast<uint8_t*>(sg.state) + at) = cv;
          if (sub == 0) {
            sg.scale[at / GROUP] = s_new;
            if (FORMAT == MMB_STATE_FP8_EXPAND) { sg.expand[at / GROUP] = ep.expand; sg.sqrt_mm[at / GROUP] = ep.sqrt_mm; }
          }
#pragma unroll
          for (int i = 0; i < ELEMS_PER_LANE; ++i) ss = fmaf(m[i], m[i], ss);
          if (sg.m_out != nullptr) {
            uint4 mv[2];
            __nv_bfloat162* mh = reinterpret_cast<__nv_bfloat162*>(mv);
#pragma unroll
            for (int i = 0; i < 8; ++i) mh[i] = __floats2bfloat162_rn(m[2 * i], m[2 * i + 1]);
            uint4* mp = reinterpret_cast<uint4*>(sg.m_out + at);
            mp[0] = mv[0];
            mp[1] = mv[1];
          }
        }
        cur = nxt;
        cur_ok = nxt_ok;
      }
    } else if (!ALL_FAST)
    for (int g0 = 0; g0 < ngroups; g0 += 4) {
      const int gi = g0 + grp_in_warp;
      const bool active = gi < ngroups;
      const long long gstart = e0 + static_cast<long long>(gi) * GROUP;  // first element of the group
      const long long at = gstart + sub * ELEMS_PER_LANE;
      int n = 0;  // valid elements of this lane
      if (active) {
        long long rem = sg.numel - at;
        n = rem >= ELEMS_PER_LANE ? ELEMS_PER_LANE : (rem > 0 ? static_cast<int>(rem) : 0);
      }
      const bool vec = sg.vec_ok && n == ELEMS_PER_LANE;
      const long long gidx = gstart / GROUP;  // group index within the tensor

      float m[ELEMS_PER_LANE];
      float g[ELEMS_PER_LANE];
#pragma unroll
      for (int i = 0; i < ELEMS_PER_LANE; ++i) { m[i] = 0.0f; g[i] = 0.0f; }

      if (n > 0) {
        Elem<GradT>::load16(sg.grad, at, vec, n, g);
        if (FORMAT == MMB_STATE_FP8_ABSMAX) {
          load_codes16(static_cast<const uint8_t*>(sg.state) + at, vec, n, m);
          const float s = sg.scale[gidx];
#pragma unroll
          for (int i = 0; i < ELEMS_PER_LANE; ++i) m[i] = __fmul_rn(m[i], s);
        } else if (FORMAT == MMB_STATE_FP8_EXPAND) {
          load_codes16(static_cast<const uint8_t*>(sg.state) + at, vec, n, m);
          const float s = sg.scale[gidx], ex = sg.expand[gidx], sq = sg.sqrt_mm[gidx];
#pragma unroll
          for (int i = 0; i < ELEMS_PER_LANE; ++i) m[i] = expand_decode<DIV>(m[i], s, ex, sq, true);
        } else if (FORMAT == MMB_STATE_BF16) {
          Elem<__nv_bfloat16>::load16(sg.state, at, vec, n, m);
        } else {
          Elem<float>::load16(sg.state, at, vec, n, m);
        }
      }

      // heavy ball: two roundings in the state's arithmetic type
      float amax = 0.0f, amin = 3.4028235e38f;
      int any_nz = 0;
#pragma unroll
      for (int i = 0; i < ELEMS_PER_LANE; ++i) {
        float gi_f = __fmul_rn(g[i], grad_scale);
        if (sizeof(GradT) == 2 && grad_scale != 1.0f) gi_f = bf16_round(gi_f);  // as grad.mul_(scale) would leave it
        float t = __fmul_rn(beta, m[i]);
        if (FORMAT == MMB_STATE_BF16) t = bf16_round(t);
        t = __fadd_rn(t, gi_f);
        if (FORMAT == MMB_STATE_BF16) t = bf16_round(t);
        if (i >= n) t = 0.0f;
        m[i] = t;
        float a = fabsf(t);
        amax = fmaxf(amax, a);
        if (FORMAT == MMB_STATE_FP8_EXPAND && a > 0.0f) { amin = fminf(amin, a); any_nz = 1; }
      }

      if (FORMAT == MMB_STATE_FP8_ABSMAX) {
        amax = group_max(amax);
        const float s_new = fdiv<DIV>(__fadd_rn(amax, 1e-20f), 448.0f);
        float q[ELEMS_PER_LANE];
#pragma unroll
        for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = fdiv<DIV>(m[i], s_new);
        if (n > 0) {
          store_codes16(static_cast<uint8_t*>(sg.state) + at, vec, n, q);
          if (sub == 0) sg.scale[gidx] = s_new;
        }
      } else if (FORMAT == MMB_STATE_FP8_EXPAND) {
        amax = group_max(amax);
        amin = group_min(amin);
        any_nz = group_or(any_nz);
        const ExpandParams p = expand_group_params<DIV>(amax, amin, any_nz != 0, expand_min);
        float q[ELEMS_PER_LANE];
#pragma unroll
        for (int i = 0; i < ELEMS_PER_LANE; ++i) q[i] = expand_normalize<DIV>(m[i], i < n, p, true);
        if (n > 0) {
          store_codes16(static_cast<uint8_t*>(sg.state) + at, vec, n, q);
          if (sub == 0) { sg.scale[gidx] = p.scale; sg.expand[gidx] = p.expand; sg.sqrt_mm[gidx] = p.sqrt_mm; }
        }
      } else if (FORMAT == MMB_STATE_BF16) {
        if (n > 0) Elem<__nv_bfloat16>::store16(sg.state, at, vec, n, m);
      } else {
        if (n > 0) Elem<float>::store16(sg.state, at, vec, n, m);
      }

      // what Newton-Schulz reads, and its squared norm
#pragma unroll
      for (int i = 0; i < ELEMS_PER_LANE; ++i) ss = fmaf(m[i], m[i], ss);
      if (n > 0 && sg.m_out != nullptr && static_cast<void*>(sg.m_out) != sg.state)
        Elem<__nv_bfloat16>::store16(sg.m_out, at, vec, n, m);
    }

#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0 && partials != nullptr) partials[sg.partial_base + blk * sg.cpb + chunk] = ss;
  }
}

// Sum each block's partials in a fixed order (lane-strided, then a tree): one
// warp per block over all blocks of the launch.
__global__ void __launch_bounds__(THREADS)
block_sumsq_kernel(const __grid_constant__ SegTable tab, const float* __restrict__ partials,
                   float* __restrict__ block_sumsq) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long total = tab.block_start[tab.nseg];
  for (long long gb = warp_global; gb < total; gb += nwarps) {
    int lo = 0, hi = tab.nseg;
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (tab.block_start[mid] <= gb) lo = mid; else hi = mid;
    }
    const SegDev& sg = tab.seg[lo];
    const long long b = gb - tab.block_start[lo];
    const float* p = partials + sg.partial_base + b * sg.cpb;
    float acc = 0.0f;
    for (int i = lane; i < sg.cpb; i += 32) acc += p[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) block_sumsq[sg.first_block + b] = acc;
  }
}

// ------------------------------------------------------- stand-alone codecs
// One warp per group of 128 (4 elements per lane); not performance critical:
// used for first-step state creation, state_dict export and tests.
template <int FORMAT, int DIV>
__global__ void __launch_bounds__(THREADS)
quantize_kernel(const float* __restrict__ value, uint8_t* __restrict__ codes, float* __restrict__ scale,
                float* __restrict__ expand, float* __restrict__ sqrt_mm, long long numel, int is_signed,
                float expand_min) {
  const int lane = threadIdx.x & 31;
  const long long ngroups = (numel + GROUP - 1) / GROUP;
  const long long warp_global = static_cast<long long>(blockIdx.x) * (THREADS / 32) + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * (THREADS / 32);
  for (long long gidx = warp_global; gidx < ngroups; gidx += nwarps) {
    float m[4];
    bool ok[4];
    float amax = 0.0f, amin = 3.4028235e38f;
    int any_nz = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      long long at = gidx * GROUP + lane * 4 + i;
      ok[i] = at < numel;
      m[i] = ok[i] ? value[at] : 0.0f;
      float a = fabsf(m[i]);
      amax = fmaxf(amax, a);
      if (ok[i] && a > 0.0f) { amin = fminf(amin, a); any_nz = 1; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      amin = fminf(amin, __shfl_xor_sync(0xffffffffu, amin, o));
      any_nz |= __shfl_xor_sync(0xffffffffu, any_nz, o);
    }
    float q[4];
    if (FORMAT == MMB_STATE_FP8_ABSMAX) {
      const float s = fdiv<DIV>(__fadd_rn(amax, 1e-20f), 448.0f);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = fdiv<DIV>(m[i], s);
      if (lane == 0) scale[gidx] = s;
    } else {
      const ExpandParams p = expand_group_params<DIV>(amax, amin, any_nz != 0, expand_min);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = expand_normalize<DIV>(m[i], ok[i], p, is_signed != 0);
      if (lane == 0) { scale[gidx] = p.scale; expand[gidx] = p.expand; sqrt_mm[gidx] = p.sqrt_mm; }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      long long at = gidx * GROUP + lane * 4 + i;
      if (ok[i]) codes[at] = static_cast<uint8_t>(float2_to_e4m3x2(q[i], 0.0f) & 0xff);
    }
  }
}

template <int FORMAT, int DIV>
__global__ void __launch_bounds__(THREADS)
dequantize_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ scale,
                  const float* __restrict__ expand, const float* __restrict__ sqrt_mm, float* __restrict__ out,
                  long long numel, int is_signed) {
  const long long stride = static_cast<long long>(gridDim.x) * THREADS;
  for (long long at = static_cast<long long>(blockIdx.x) * THREADS + threadIdx.x; at < numel; at += stride) {
    const long long gidx = at / GROUP;
    const float raw = e4m3x2_to_float2(codes[at]).x;
    if (FORMAT == MMB_STATE_FP8_ABSMAX)
      out[at] = __fmul_rn(raw, scale[gidx]);
    else
      out[at] = expand_decode<DIV>(raw, scale[gidx], expand[gidx], sqrt_mm[gidx], is_signed != 0);
  }
}

// ------------------------------------------------------------------- host
struct Plan {
  long long cpb;          // partials per block
  long long nblocks;
  long long block_elems;  // effective (== numel when blocks do not hold whole groups)
};

Plan plan_segment(const mmb_momentum_seg& s) {
  Plan p;
  p.block_elems = s.block_elems;
  if (p.block_elems <= 0 || p.block_elems % GROUP != 0 || s.numel % p.block_elems != 0) p.block_elems = s.numel;
  p.nblocks = s.numel / p.block_elems;
  p.cpb = (p.block_elems + UNIT - 1) / UNIT;
  return p;
}

template <int FORMAT, typename GradT>
void launch_momentum(int div_mode, bool all_fast, const SegTable& tab, int grid, float beta, float grad_scale,
                     float expand_min, float* partials, cudaStream_t st) {
  if (FORMAT == MMB_STATE_FP8_ABSMAX && all_fast) {
    if (div_mode == MMB_DIV_IEEE)
      launch_stream_kernel(momentum_kernel<MMB_STATE_FP8_ABSMAX, GradT, MMB_DIV_IEEE, true>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
    else if (div_mode == MMB_DIV_IEEE_STRICT)
      launch_stream_kernel(momentum_kernel<MMB_STATE_FP8_ABSMAX, GradT, MMB_DIV_IEEE_STRICT, true>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
    else
      launch_stream_kernel(momentum_kernel<MMB_STATE_FP8_ABSMAX, GradT, MMB_DIV_FULL, true>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
    return;
  }
  if ((FORMAT == MMB_STATE_BF16 || FORMAT == MMB_STATE_F32) && all_fast) {
    launch_stream_kernel(momentum_kernel<FORMAT, GradT, MMB_DIV_IEEE, true>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
    return;
  }
  if (FORMAT == MMB_STATE_FP8_EXPAND && all_fast) {
    if (div_mode == MMB_DIV_IEEE_STRICT)
      launch_stream_kernel(momentum_kernel<MMB_STATE_FP8_EXPAND, GradT, MMB_DIV_IEEE_STRICT, true>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
    else if (div_mode != MMB_DIV_FULL)
      launch_stream_kernel(momentum_kernel<MMB_STATE_FP8_EXPAND, GradT, MMB_DIV_IEEE, true>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
    else
      launch_stream_kernel(momentum_kernel<MMB_STATE_FP8_EXPAND, GradT, MMB_DIV_FULL, true>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
    return;
  }
  if (div_mode != MMB_DIV_FULL)
    launch_stream_kernel(momentum_kernel<FORMAT, GradT, MMB_DIV_IEEE, false>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
  else
    launch_stream_kernel(momentum_kernel<FORMAT, GradT, MMB_DIV_FULL, false>, grid, THREADS, st, tab, beta, grad_scale, expand_min, partials, device_grad_scale());
}

template <typename GradT>
void launch_momentum_format(int format, int div_mode, bool all_fast, const SegTable& tab, int grid, float beta,
                            float grad_scale, float expand_min, float* partials, cudaStream_t st) {
  switch (format) {
    case MMB_STATE_FP8_ABSMAX:
      launch_momentum<MMB_STATE_FP8_ABSMAX, GradT>(div_mode, all_fast, tab, grid, beta, grad_scale, expand_min, partials, st);
      break;
    case MMB_STATE_FP8_EXPAND:
      launch_momentum<MMB_STATE_FP8_EXPAND, GradT>(div_mode, all_fast, tab, grid, beta, grad_scale, expand_min, partials, st);
      break;
    case MMB_STATE_BF16:
      launch_momentum<MMB_STATE_BF16, GradT>(MMB_DIV_IEEE, all_fast, tab, grid, beta, grad_scale, expand_min, partials, st);
      break;
    default:
      launch_momentum<MMB_STATE_F32, GradT>(MMB_DIV_IEEE, all_fast, tab, grid, beta, grad_scale, expand_min, partials, st);
      break;
  }
}

}  // namespace

int momentum_step_impl(const char* who, const mmb_momentum_seg* segs, int nseg, int grad_dtype, int state_format,
                       int div_mode, float beta, float grad_scale, int expand_min, float* block_sumsq_dev,
                       float* scratch_dev, int64_t scratch_floats, void* stream) {
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "%s: bad segment table", who);
  MMB_REQUIRE(grad_dtype == MMB_BF16 || grad_dtype == MMB_F32, "%s: grad_dtype %d", who, grad_dtype);
  MMB_REQUIRE(state_format >= MMB_STATE_FP8_ABSMAX && state_format <= MMB_STATE_F32,
              "%s: state_format %d", who, state_format);
  MMB_REQUIRE(div_mode >= MMB_DIV_IEEE && div_mode <= MMB_DIV_IEEE_STRICT, "%s: div_mode %d", who, div_mode);
  if (nseg == 0) return MMB_OK;
  const int64_t need = mmb_momentum_scratch_floats(segs, nseg);
  if (block_sumsq_dev != nullptr)
    MMB_REQUIRE(scratch_dev != nullptr && scratch_floats >= need,
                "%s: scratch of %lld floats needed, %lld given", who, (long long)need,
                (long long)scratch_floats);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "%s: no CUDA device", who);
  float* partials = block_sumsq_dev != nullptr ? scratch_dev : nullptr;

  long long partial_base = 0;
  for (int base = 0; base < nseg; base += MAX_SEG) {
    SegTable tab;
    tab.nseg = (nseg - base) < MAX_SEG ? (nseg - base) : MAX_SEG;
    long long units = 0, blocks = 0;
    bool all_fast = true;
    for (int i = 0; i < tab.nseg; ++i) {
      const mmb_momentum_seg& s = segs[base + i];
      MMB_REQUIRE(s.numel > 0 && s.grad != nullptr && s.state != nullptr, "%s: segment %d empty", who,
                  base + i);
      if (state_format == MMB_STATE_FP8_ABSMAX || state_format == MMB_STATE_FP8_EXPAND)
        MMB_REQUIRE(s.scale != nullptr, "%s: segment %d has no scale array", who, base + i);
      if (state_format == MMB_STATE_FP8_EXPAND)
        MMB_REQUIRE(s.expand != nullptr && s.sqrt_minmax != nullptr,
                    "%s: segment %d lacks expand/sqrt_minmax", who, base + i);
      const Plan p = plan_segment(s);
      if (block_sumsq_dev != nullptr)
        MMB_REQUIRE(p.block_elems == s.block_elems,
                    "%s: block_elems %lld of segment %d must be a multiple of 128 dividing numel "
                    "when block sums are requested", who, (long long)s.block_elems, base + i);
      SegDev& d = tab.seg[i];
      d.grad = s.grad;
      d.state = s.state;
      d.scale = s.scale;
      d.expand = s.expand;
      d.sqrt_mm = s.sqrt_minmax;
      d.m_out = static_cast<__nv_bfloat16*>(s.m_bf16);
      d.numel = s.numel;
      d.block_elems = p.block_elems;
      d.partial_base = partial_base;
      d.first_block = s.first_block;
      d.cpb = static_cast<int>(p.cpb);
      d.vec_ok = aligned16(s.grad) && aligned16(s.state) && (s.m_bf16 == nullptr || aligned16(s.m_bf16));
      all_fast = all_fast && d.vec_ok && (s.numel % GROUP) == 0;
      tab.unit_start[i] = units;
      tab.block_start[i] = blocks;
      blocks += p.nblocks;
      units += p.nblocks * p.cpb;
      partial_base += p.nblocks * p.cpb;
    }
    tab.unit_start[tab.nseg] = units;
    tab.block_start[tab.nseg] = blocks;
    const long long warps_per_cta = stream_threads(THREADS) / 32;
    long long want = (units + warps_per_cta - 1) / warps_per_cta;
    long long cap = stream_grid_cap(sms);  // a few waves of 8 resident CTAs per SM unless capped
    int grid = static_cast<int>(want < cap ? want : cap);
    if (grid < 1) grid = 1;
    if (grad_dtype == MMB_BF16)
      launch_momentum_format<__nv_bfloat16>(state_format, div_mode, all_fast, tab, grid, beta, grad_scale,
                                            static_cast<float>(expand_min), partials, st);
    else
      launch_momentum_format<float>(state_format, div_mode, all_fast, tab, grid, beta, grad_scale,
                                    static_cast<float>(expand_min), partials, st);
    MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
    if (block_sumsq_dev != nullptr) {
      long long g2 = (blocks + warps_per_cta - 1) / warps_per_cta;
      if (g2 > sms * 4) g2 = sms * 4;
      if (g2 < 1) g2 = 1;
      launch_stream_kernel(block_sumsq_kernel, static_cast<int>(g2), THREADS, st, tab, partials, block_sumsq_dev);
      MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
    }
  }
  return MMB_OK;
}

}  // namespace mmb

// ------------------------------------------------ scratch that needs no allocator
// Per-chunk partial sums for mmb_momentum_step_static().  A file-scope device
// array: every GPU that loads this library carries these 4 MiB until the
// process exits, and no allocator is involved in getting it.
constexpr long long STATIC_SCRATCH_FLOATS = 1ll << 20;  // 4096 elements per partial -> 2^32 state elements
static __device__ __align__(256) float g_static_partials[STATIC_SCRATCH_FLOATS];

namespace mmb {
namespace {
constexpr int MAX_DEVICES = 64;
// One slot per device ordinal, filled on the first call on that device.  Atomic because two host threads may
// make that first call at once (both then store the same address).
std::atomic<float*> g_static_partials_addr[MAX_DEVICES];

// In host code `g_static_partials` is only a handle for the runtime, not a
// device address; the address on the current device has to be asked for.
int static_partials_for_current_device(float** out) {
  int dev = -1;
  MMB_CUDA_CHECK(cudaGetDevice(&dev));
  MMB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "mmb_momentum_step_static: device index %d not supported", dev);
  float* cached = g_static_partials_addr[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* p = nullptr;
    MMB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_partials));
    cached = static_cast<float*>(p);
    g_static_partials_addr[dev].store(cached, std::memory_order_release);
  }
  *out = cached;
  return MMB_OK;
}
}  // namespace
}  // namespace mmb

extern "C" {

int64_t mmb_momentum_scratch_floats(const mmb_momentum_seg* segs, int nseg) {
  int64_t total = 0;
  for (int i = 0; i < nseg; ++i) {
    if (segs[i].numel <= 0) continue;
    mmb::Plan p = mmb::plan_segment(segs[i]);
    total += p.nblocks * p.cpb;
  }
  return total;
}

int mmb_momentum_step(const mmb_momentum_seg* segs, int nseg, int grad_dtype, int state_format, int div_mode,
                      float beta, float grad_scale, int expand_min, float* block_sumsq_dev, float* scratch_dev,
                      int64_t scratch_floats, void* stream) {
  return mmb::momentum_step_impl("mmb_momentum_step", segs, nseg, grad_dtype, state_format, div_mode, beta, grad_scale,
                                 expand_min, block_sumsq_dev, scratch_dev, scratch_floats, stream);
}

int64_t mmb_momentum_static_max_floats(void) { return STATIC_SCRATCH_FLOATS; }

int mmb_momentum_step_static(const mmb_momentum_seg* segs, int nseg, int grad_dtype, int state_format, int div_mode,
                             float beta, float grad_scale, int expand_min, float* block_sumsq_dev, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(nseg >= 0 && (nseg == 0 || segs != nullptr), "mmb_momentum_step_static: bad segment table");
  const int64_t need = mmb_momentum_scratch_floats(segs, nseg);
  MMB_REQUIRE(need <= STATIC_SCRATCH_FLOATS,
              "mmb_momentum_step_static: this table needs %lld partial sums but the built-in scratch holds %lld "
              "(about 4.29e9 state elements); split the table or use mmb_momentum_step with your own scratch",
              (long long)need, (long long)STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  int rc = static_partials_for_current_device(&scratch);
  if (rc != MMB_OK) return rc;
  return momentum_step_impl("mmb_momentum_step_static", segs, nseg, grad_dtype, state_format, div_mode, beta,
                            grad_scale, expand_min, block_sumsq_dev, scratch, STATIC_SCRATCH_FLOATS, stream);
}

int mmb_fp8_quantize(const float* value_dev, uint8_t* codes_dev, float* scale_dev, float* expand_dev,
                     float* sqrt_minmax_dev, int64_t numel, int state_format, int is_signed, int div_mode,
                     int expand_min, void* stream) {
  using namespace mmb;
  MMB_REQUIRE(state_format == MMB_STATE_FP8_ABSMAX || state_format == MMB_STATE_FP8_EXPAND,
              "mmb_fp8_quantize: state_format %d", state_format);
  MMB_REQUIRE(numel >= 0 && (numel == 0 || (value_dev && codes_dev && scale_dev)), "mmb_fp8_quantize: null pointer");
  if (state_format == MMB_STATE_FP8_EXPAND)
    MMB_REQUIRE(numel == 0 || (expand_dev && sqrt_minmax_dev), "mmb_fp8_quantize: expansion arrays missing");
  if (numel == 0) return MMB_OK;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_fp8_quantize: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long groups = (numel + GROUP - 1) / GROUP;
  long long want = (groups + THREADS / 32 - 1) / (THREADS / 32);
  int grid = static_cast<int>(want < sms * 32LL ? want : sms * 32LL);
  const float em = static_cast<float>(expand_min);
#define MMB_Q(F, D) \
  quantize_kernel<F, D><<<grid, THREADS, 0, st>>>(value_dev, codes_dev, scale_dev, expand_dev, sqrt_minmax_dev, numel, is_signed, em)
  if (state_format == MMB_STATE_FP8_ABSMAX) {
    if (div_mode != MMB_DIV_FULL) MMB_Q(MMB_STATE_FP8_ABSMAX, MMB_DIV_IEEE); else MMB_Q(MMB_STATE_FP8_ABSMAX, MMB_DIV_FULL);
  } else {
    if (div_mode != MMB_DIV_FULL) MMB_Q(MMB_STATE_FP8_EXPAND, MMB_DIV_IEEE); else MMB_Q(MMB_STATE_FP8_EXPAND, MMB_DIV_FULL);
  }
#undef MMB_Q
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

int mmb_fp8_dequantize(const uint8_t* codes_dev, const float* scale_dev, const float* expand_dev,
                       const float* sqrt_minmax_dev, float* out_dev, int64_t numel, int state_format, int is_signed,
                       void* stream) {
  using namespace mmb;
  MMB_REQUIRE(state_format == MMB_STATE_FP8_ABSMAX || state_format == MMB_STATE_FP8_EXPAND,
              "mmb_fp8_dequantize: state_format %d", state_format);
  MMB_REQUIRE(numel >= 0 && (numel == 0 || (codes_dev && scale_dev && out_dev)), "mmb_fp8_dequantize: null pointer");
  if (state_format == MMB_STATE_FP8_EXPAND)
    MMB_REQUIRE(numel == 0 || (expand_dev && sqrt_minmax_dev), "mmb_fp8_dequantize: expansion arrays missing");
  if (numel == 0) return MMB_OK;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_fp8_dequantize: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  long long want = (numel + THREADS - 1) / THREADS;
  int grid = static_cast<int>(want < sms * 32LL ? want : sms * 32LL);
  if (state_format == MMB_STATE_FP8_ABSMAX)
    dequantize_kernel<MMB_STATE_FP8_ABSMAX, MMB_DIV_IEEE><<<grid, THREADS, 0, st>>>(codes_dev, scale_dev, expand_dev,
                                                                                  sqrt_minmax_dev, out_dev, numel, is_signed);
  else
    dequantize_kernel<MMB_STATE_FP8_EXPAND, MMB_DIV_IEEE><<<grid, THREADS, 0, st>>>(codes_dev, scale_dev, expand_dev,
                                                                                  sqrt_minmax_dev, out_dev, numel, is_signed);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

}  // extern "C"
