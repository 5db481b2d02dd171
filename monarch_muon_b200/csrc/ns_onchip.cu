// Newton-Schulz for small blocks, entirely on chip: one CTA per block, one launch for all five iterations.
//
// For a block whose short side m is at most 128 and whose long side n is at most 384, the block X, the
// Gram matrix Ah and the polynomial Pp fit one SM: X (<= 96 KiB), Ah and Pp (32 KiB each) stay in shared
// memory as bf16, the accumulators in tensor memory, and the fifteen GEMMs of the iteration
//     Ah = s^2 X X^T + beta I ;  Pp = c Ah Ah + kappa I ;  X = s Pp X          (s: first iteration only)
// run back to back without touching global memory (the multi-launch path in newton_schulz.cu round-trips
// every intermediate through L2/HBM and pays fifteen launches per shape group).  Same arithmetic: bf16
// operands, fp32 accumulation in tcgen05.mma, every intermediate rounded to bf16.
//
// Layout.  The stored block [rows][cols] is held as tiles of 128 rows x 64 columns (128-byte rows, 128-byte
// swizzle), tile (rt, ct) at (rt * col_tiles + ct) * 16 KiB, loaded by TMA with zero fill beyond the edges.
// One tile serves every role it has: a K-major operand tile [128 rows][64 k] for X X^T (wide) and Y Pp
// (tall), and the two 64-k halves of an MN-major operand for Pp X (wide) and Y^T Y (tall) - tcgen05 takes
// the major-ness per instruction, so nothing is ever transposed.  Ah and Pp are two tiles each.
//
// One warp group of 128 threads: thread 0 issues TMA and MMAs, all four warps drain tensor memory
// (thread t owns row t), convert and write the next operand into shared memory.  Phases are serial -
// the block is too small for overlap inside a CTA to matter; parallelism comes from one block per SM.
// Every wait is bounded and reports through the device status word.
//
// Second kernel, same scheme, for wide or square blocks with 128 < rows <= 256 and cols <= 256 (the 256 x 256
// blocks of a 1024-wide model with four blocks): X is two row blocks of 128 (eight tiles, 128 KiB); Ah and
// Pp are symmetric and share ONE buffer that holds only the 128 x 128 blocks (0,0), (0,1), (1,1) (six tiles,
// 96 KiB) - block (1,0) is read from block (0,1) through an MN-major descriptor, and Pp overwrites Ah once
// every product that reads Ah has completed (all three result blocks wait in tensor memory meanwhile).
#include "common.cuh"
#include "gemm.cuh"
#include "tcgen05_ptx.cuh"

namespace mmb {
namespace tc {

constexpr int OC_THREADS = 128;
constexpr int OC_TILE_BYTES = 128 * 128;   // 128 rows x 64 bf16
constexpr int OC_MAX_X_TILES = 6;          // 128 x 384 or 384 x 128
constexpr int OC_X_BYTES = OC_MAX_X_TILES * OC_TILE_BYTES;
constexpr int OC_SMEM_BYTES = OC_X_BYTES + 4 * OC_TILE_BYTES + 1024 /*align*/ + 64 /*barriers*/;
constexpr int OC_TMEM_COLS = 512;
constexpr int OC_ACC_SMALL = 384;          // column of the Gram / Poly accumulator; the Apply result uses [0, 384)

struct OnchipArgs {
  int batch, rows, cols;
  int tall;          // rows > cols
  int row_tiles;     // ceil(rows / 128)
  int col_tiles;     // ceil(cols / 64); 2 for the short side when tall
  const float* inv_norm;
  float beta, kappa, c;
  __nv_bfloat16* out;      // [batch][rows][cols], or null with upd_w
  void* const* upd_w;      // fused update: W[b] <- W[b] + upd_alpha * result
  float upd_alpha;
  int upd_f32;
  int32_t* status;
  long long wait_limit;
};

// descriptor halves (see gemm_tcgen05.cu): high = stride offset 1024 | version 1 | 128-byte swizzle
constexpr uint32_t OC_DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t OC_LBO_TILE = OC_TILE_BYTES >> 4;   // MN-major: the next 64 rows are the next tile

__device__ __forceinline__ uint32_t oc_idesc(int n, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}
// One K=64 slice as four K=16 instructions.  K-major operands advance 32 bytes per instruction,
// MN-major ones 16 rows of 128 bytes.
__device__ __forceinline__ void oc_mma_slice(uint32_t d_tmem, uint32_t a_addr, bool a_mn, uint32_t b_addr, bool b_mn,
                                             int n, uint32_t& accumulate) {
  const uint32_t idesc = oc_idesc(n, a_mn, b_mn);
  const uint32_t a_lo = (a_addr >> 4) | ((a_mn ? OC_LBO_TILE : 1u) << 16);
  const uint32_t b_lo = (b_addr >> 4) | ((b_mn ? OC_LBO_TILE : 1u) << 16);
  const uint32_t a_step = a_mn ? (16u * 128u) >> 4 : 32u >> 4;
  const uint32_t b_step = b_mn ? (16u * 128u) >> 4 : 32u >> 4;
#pragma unroll
  for (uint32_t k = 0; k < 4; ++k) {
    tcgen05_mma_f16_split<false>(d_tmem, a_lo + k * a_step, OC_DESC_HI, b_lo + k * b_step, OC_DESC_HI, idesc, accumulate);
    accumulate = 1u;
  }
}

// Thread `row` drains `groups` x 32 accumulator columns starting at column acc_col, scales them, adds
// `diag` on the diagonal (column index == diag_col0 + row, rows below diag_rows only), rounds to bf16 and
// writes them as row `row` of consecutive 64-column tiles starting at dst (tiles OC_TILE_BYTES apart).
__device__ __forceinline__ void oc_drain(uint32_t tmem_row_base, int acc_col, int groups, uint8_t* dst, int row,
                                         float scale, float diag, int diag_rows) {
#pragma unroll 1
  for (int g = 0; g < groups; ++g) {
    uint32_t v[32];
    tcgen05_ld_32x32b_x32(tmem_row_base + acc_col + 32 * g, v);
    tcgen05_wait_ld();
    uint8_t* tile_row = dst + (g >> 1) * OC_TILE_BYTES + row * 128;
    const int dcol = row - 32 * g;   // position of the diagonal element inside this group, if any
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = 8 * u + 2 * i;
        float x0 = scale * __uint_as_float(v[e]);
        float x1 = scale * __uint_as_float(v[e + 1]);
        if (row < diag_rows) {
          if (e == dcol) x0 += diag;
          if (e + 1 == dcol) x1 += diag;
        }
        oh[i] = __floats2bfloat162_rn(x0, x1);
      }
      const int q = (g & 1) * 4 + u;   // 16-byte unit inside the 128-byte row
      *reinterpret_cast<uint4*>(tile_row + ((q ^ (row & 7)) << 4)) = o;
    }
  }
}

// The finished block, held as tiles in shared memory, goes to `out` or is applied to the weights:
// coalesced 16-byte units, W <- fma(alpha, result, W) with one rounding to the weights' type.
__device__ __forceinline__ void oc_store_result(const OnchipArgs& args, const uint8_t* x_ptr, int b, int tid) {
  const int units_per_row = args.cols >> 3;   // 16-byte units
  const long long units = static_cast<long long>(args.rows) * units_per_row;
  const long long blk = static_cast<long long>(args.rows) * args.cols;
  for (long long u = tid; u < units; u += OC_THREADS) {
    const int row = static_cast<int>(u / units_per_row);
    const int col = static_cast<int>(u - static_cast<long long>(row) * units_per_row) << 3;
    const int r = row & 127, q = (col & 63) >> 3;
    const uint8_t* tile = x_ptr + ((row >> 7) * args.col_tiles + (col >> 6)) * OC_TILE_BYTES;
    const uint4 ov = *reinterpret_cast<const uint4*>(tile + r * 128 + ((q ^ (r & 7)) << 4));
    const long long at = static_cast<long long>(row) * args.cols + col;
    if (args.upd_w == nullptr) {
      *reinterpret_cast<uint4*>(args.out + static_cast<long long>(b) * blk + at) = ov;
    } else {
      const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&ov);
      if (args.upd_f32) {
        float4* wp = reinterpret_cast<float4*>(static_cast<float*>(args.upd_w[b]) + at);
        float4 w0 = wp[0], w1 = wp[1];
        const float2 o0 = __bfloat1622float2(oh[0]), o1 = __bfloat1622float2(oh[1]);
        const float2 o2 = __bfloat1622float2(oh[2]), o3 = __bfloat1622float2(oh[3]);
        w0.x = fmaf(args.upd_alpha, o0.x, w0.x); w0.y = fmaf(args.upd_alpha, o0.y, w0.y);
        w0.z = fmaf(args.upd_alpha, o1.x, w0.z); w0.w = fmaf(args.upd_alpha, o1.y, w0.w);
        w1.x = fmaf(args.upd_alpha, o2.x, w1.x); w1.y = fmaf(args.upd_alpha, o2.y, w1.y);
        w1.z = fmaf(args.upd_alpha, o3.x, w1.z); w1.w = fmaf(args.upd_alpha, o3.y, w1.w);
        wp[0] = w0;
        wp[1] = w1;
      } else {
        uint4* wp = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.upd_w[b]) + at);
        uint4 wv = *wp;
        __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&wv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 o = __bfloat1622float2(oh[i]);
          const float2 w = __bfloat1622float2(wh[i]);
          wh[i] = __floats2bfloat162_rn(fmaf(args.upd_alpha, o.x, w.x), fmaf(args.upd_alpha, o.y, w.y));
        }
        *wp = wv;
      }
    }
  }
}

__global__ void __launch_bounds__(OC_THREADS, 1)
ns_onchip_kernel(const __grid_constant__ CUtensorMap map_x, const OnchipArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t x_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* x_ptr = smem_raw + (x_addr - raw_addr);
  const uint32_t ah_addr = x_addr + OC_X_BYTES;
  uint8_t* ah_ptr = x_ptr + OC_X_BYTES;
  const uint32_t pp_addr = ah_addr + 2 * OC_TILE_BYTES;
  uint8_t* pp_ptr = ah_ptr + 2 * OC_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(pp_ptr + 2 * OC_TILE_BYTES);
  const uint32_t tma_bar = pp_addr + 2 * OC_TILE_BYTES;
  const uint32_t mma_bar = tma_bar + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  if (tid == 0) {
    mbar_init(tma_bar, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(OC_TMEM_COLS))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);  // this warp's 32 lanes

  const int m = args.tall ? args.cols : args.rows;
  const int x_tiles = args.row_tiles * args.col_tiles;
  uint32_t tma_phase = 0, mma_phase = 0;
  bool ok = true;

  // wait for the MMAs committed last, by every thread
  // (the verdict is made uniform over the CTA, so that all threads leave the loops together)
  auto wait_mma = [&]() {
    const bool mine = mbar_wait(mma_bar, mma_phase, abort_flag, args.status, STATUS_WAIT_EPI_TMEM_FULL, args.wait_limit);
    ok = __syncthreads_and(mine ? 1 : 0) != 0;
    mma_phase ^= 1u;
    tcgen05_fence_after();
  };
  // operands written by this thread become visible to the tensor core's reads; then everyone meets
  auto publish = [&]() {
    tcgen05_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
  };

  for (int b = blockIdx.x; b < args.batch && ok; b += gridDim.x) {
    // ---------------------------------------------------------------- load the block
    if (tid == 0) {
      mbar_expect_tx(tma_bar, static_cast<uint32_t>(x_tiles) * OC_TILE_BYTES);
      for (int rt = 0; rt < args.row_tiles; ++rt)
        for (int ct = 0; ct < args.col_tiles; ++ct)
          tma_load_3d(x_addr + (rt * args.col_tiles + ct) * OC_TILE_BYTES, &map_x, tma_bar, 64 * ct, 128 * rt, b);
    }
    {
      const bool mine = mbar_wait(tma_bar, tma_phase, abort_flag, args.status, STATUS_WAIT_MMA_FULL, args.wait_limit);
      ok = __syncthreads_and(mine ? 1 : 0) != 0;
      tma_phase ^= 1u;
    }
    if (!ok) break;
    const float s = args.inv_norm[b];

    for (int it = 0; it < 5 && ok; ++it) {
      const bool first = it == 0;
      // ------------------------------------------------------------ Gram: Ah = s^2 X X^T + beta I
      if (tid == 0) {
        tcgen05_fence_after();
        uint32_t acc = 0;
        if (!args.tall) {
          for (int ct = 0; ct < args.col_tiles; ++ct) {   // contraction over the columns, 64 at a time
            const uint32_t t = x_addr + ct * OC_TILE_BYTES;
            oc_mma_slice(tmem_base + OC_ACC_SMALL, t, false, t, false, 128, acc);
          }
        } else {
          for (int rt = 0; rt < args.row_tiles; ++rt)     // contraction over the rows: MN-major on both sides
            for (int h = 0; h < 2; ++h) {
              const uint32_t t = x_addr + rt * 2 * OC_TILE_BYTES + h * (OC_TILE_BYTES / 2);
              oc_mma_slice(tmem_base + OC_ACC_SMALL, t, true, t, true, 128, acc);
            }
        }
        tcgen05_commit(mma_bar);
      }
      wait_mma();
      if (!ok) break;
      oc_drain(tmem_row, OC_ACC_SMALL, 4, ah_ptr, tid, first ? s * s : 1.0f, args.beta, m);
      publish();
      // ------------------------------------------------------------ Poly: Pp = c Ah Ah + kappa I
      if (tid == 0) {
        tcgen05_fence_after();
        uint32_t acc = 0;
        for (int j = 0; j < 2; ++j) {
          const uint32_t t = ah_addr + j * OC_TILE_BYTES;
          oc_mma_slice(tmem_base + OC_ACC_SMALL, t, false, t, false, 128, acc);   // Ah is symmetric: B = Ah rows
        }
        tcgen05_commit(mma_bar);
      }
      wait_mma();
      if (!ok) break;
      oc_drain(tmem_row, OC_ACC_SMALL, 4, pp_ptr, tid, args.c, args.kappa, m);
      publish();
      // ------------------------------------------------------------ Apply: X = s Pp X  (tall: Y = s Y Pp)
      if (tid == 0) {
        tcgen05_fence_after();
        if (!args.tall) {
          for (int c0 = 0; c0 < args.col_tiles; c0 += 4) {            // up to 256 result columns per instruction
            const int nt = (args.col_tiles - c0) < 4 ? (args.col_tiles - c0) : 4;
            uint32_t acc = 0;
            for (int j = 0; j < 2; ++j)                                 // contraction over m, 64 at a time
              oc_mma_slice(tmem_base + 64 * c0, pp_addr + j * OC_TILE_BYTES, false,
                           x_addr + c0 * OC_TILE_BYTES + j * (OC_TILE_BYTES / 2), true, 64 * nt, acc);
          }
        } else {
          for (int rt = 0; rt < args.row_tiles; ++rt) {
            uint32_t acc = 0;
            for (int j = 0; j < 2; ++j)
              oc_mma_slice(tmem_base + 128 * rt, x_addr + (rt * 2 + j) * OC_TILE_BYTES, false,
                           pp_addr + j * OC_TILE_BYTES, false, 128, acc);
          }
        }
        tcgen05_commit(mma_bar);
      }
      wait_mma();   // every MMA that read X has finished: X may be overwritten
      if (!ok) break;
      if (!args.tall) {
        oc_drain(tmem_row, 0, 2 * args.col_tiles, x_ptr, tid, first ? s : 1.0f, 0.0f, 0);
      } else {
        for (int rt = 0; rt < args.row_tiles; ++rt)
          oc_drain(tmem_row, 128 * rt, 4, x_ptr + rt * 2 * OC_TILE_BYTES, tid, first ? s : 1.0f, 0.0f, 0);
      }
      publish();
    }
    if (!ok) break;

    // ---------------------------------------------------------------- result: store, or update the weights
    oc_store_result(args, x_ptr, b, tid);
    __syncthreads();   // the tiles are free for the next block's TMA loads
  }

  // ------------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) __nanosleep(1000);   // let bulk copies already issued land
    __syncthreads();
  }
  if (warp == 0) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(OC_TMEM_COLS))
                 : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Wide or square blocks with 128 < rows <= 256, cols <= 256.
constexpr int OC2_X_TILES = 8;             // two row blocks x four column tiles
constexpr int OC2_S_TILES = 6;             // blocks (0,0), (0,1), (1,1) of the symmetric matrix, two tiles each
constexpr int OC2_SMEM_BYTES = (OC2_X_TILES + OC2_S_TILES) * OC_TILE_BYTES + 1024 /*align*/ + 64 /*barriers*/;

// Block (i, k) of the symmetric matrix as an operand with 128 rows (MN) and the K slice `slice` (64 wide) of
// block k's index range: stored blocks are read K-major from tile `slice`; block (1,0) is the transpose of
// the stored block (0,1) and is read MN-major, K running over that block's rows.
__device__ __forceinline__ void oc2_sym_operand(uint32_t s_addr, int i, int k, int slice, uint32_t& addr, bool& mn) {
  if (i <= k) {
    const int idx = i + k;                 // (0,0) -> 0, (0,1) -> 1, (1,1) -> 2
    addr = s_addr + (2 * idx + slice) * OC_TILE_BYTES;
    mn = false;
  } else {
    addr = s_addr + 2 * OC_TILE_BYTES + slice * (OC_TILE_BYTES / 2);
    mn = true;
  }
}

__global__ void __launch_bounds__(OC_THREADS, 1)
ns_onchip2_kernel(const __grid_constant__ CUtensorMap map_x, const OnchipArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t x_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* x_ptr = smem_raw + (x_addr - raw_addr);
  const uint32_t s_addr = x_addr + OC2_X_TILES * OC_TILE_BYTES;
  uint8_t* s_ptr = x_ptr + OC2_X_TILES * OC_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_ptr + OC2_S_TILES * OC_TILE_BYTES);
  const uint32_t tma_bar = s_addr + OC2_S_TILES * OC_TILE_BYTES;
  const uint32_t mma_bar = tma_bar + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  if (tid == 0) {
    mbar_init(tma_bar, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(static_cast<uint32_t>(OC_TMEM_COLS))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

  const int m = args.rows;                       // wide or square: the short side is the rows
  const int ct_n = args.col_tiles;               // 64-column tiles of X (<= 4)
  const int x_tiles = 2 * ct_n;
  const int rows_in_block[2] = {128, m - 128};   // rows of each row block that exist (the rest is zero fill)
  uint32_t tma_phase = 0, mma_phase = 0;
  bool ok = true;

  auto wait_mma = [&]() {
    const bool mine = mbar_wait(mma_bar, mma_phase, abort_flag, args.status, STATUS_WAIT_EPI_TMEM_FULL, args.wait_limit);
    ok = __syncthreads_and(mine ? 1 : 0) != 0;
    mma_phase ^= 1u;
    tcgen05_fence_after();
  };
  auto publish = [&]() {
    tcgen05_fence_before();
    fence_proxy_async_smem();
    __syncthreads();
  };
  // the three stored blocks of a symmetric result wait at tensor-memory columns 0, 128, 256; thread `tid` owns row tid
  auto drain_sym = [&](float scale, float diag) {
    oc_drain(tmem_row, 0, 4, s_ptr, tid, scale, diag, rows_in_block[0]);                          // (0,0)
    oc_drain(tmem_row, 128, 4, s_ptr + 2 * OC_TILE_BYTES, tid, scale, 0.0f, 0);                   // (0,1)
    oc_drain(tmem_row, 256, 4, s_ptr + 4 * OC_TILE_BYTES, tid, scale, diag, rows_in_block[1]);    // (1,1)
  };

  for (int b = blockIdx.x; b < args.batch && ok; b += gridDim.x) {
    if (tid == 0) {
      mbar_expect_tx(tma_bar, static_cast<uint32_t>(x_tiles) * OC_TILE_BYTES);
      for (int rt = 0; rt < 2; ++rt)
        for (int ct = 0; ct < ct_n; ++ct)
          tma_load_3d(x_addr + (rt * ct_n + ct) * OC_TILE_BYTES, &map_x, tma_bar, 64 * ct, 128 * rt, b);
    }
    {
      const bool mine = mbar_wait(tma_bar, tma_phase, abort_flag, args.status, STATUS_WAIT_MMA_FULL, args.wait_limit);
      ok = __syncthreads_and(mine ? 1 : 0) != 0;
      tma_phase ^= 1u;
    }
    if (!ok) break;
    const float s = args.inv_norm[b];

    for (int it = 0; it < 5 && ok; ++it) {
      const bool first = it == 0;
      // ------------------------------------------------------------ Gram: Ah(i,j) = s^2 X_i X_j^T (+ beta I)
      if (tid == 0) {
        tcgen05_fence_after();
        for (int idx = 0; idx < 3; ++idx) {
          const int i = idx >> 1, j = (idx + 1) >> 1;            // (0,0), (0,1), (1,1)
          uint32_t acc = 0;
          for (int ct = 0; ct < ct_n; ++ct)
            oc_mma_slice(tmem_base + 128 * idx, x_addr + (i * ct_n + ct) * OC_TILE_BYTES, false,
                         x_addr + (j * ct_n + ct) * OC_TILE_BYTES, false, 128, acc);
        }
        tcgen05_commit(mma_bar);
      }
      wait_mma();
      if (!ok) break;
      drain_sym(first ? s * s : 1.0f, args.beta);
      publish();
      // ------------------------------------------------------------ Poly: Pp(i,j) = c sum_k Ah(i,k) Ah(j,k)^T (+ kappa I)
      if (tid == 0) {
        tcgen05_fence_after();
        for (int idx = 0; idx < 3; ++idx) {
          const int i = idx >> 1, j = (idx + 1) >> 1;
          uint32_t acc = 0;
          for (int k = 0; k < 2; ++k)
            for (int slice = 0; slice < 2; ++slice) {
              uint32_t a_addr, b_addr;
              bool a_mn, b_mn;
              oc2_sym_operand(s_addr, i, k, slice, a_addr, a_mn);
              oc2_sym_operand(s_addr, j, k, slice, b_addr, b_mn);
              oc_mma_slice(tmem_base + 128 * idx, a_addr, a_mn, b_addr, b_mn, 128, acc);
            }
        }
        tcgen05_commit(mma_bar);
      }
      wait_mma();   // every product that read Ah has completed: the buffer may take Pp
      if (!ok) break;
      drain_sym(args.c, args.kappa);
      publish();
      // ------------------------------------------------------------ Apply: X_i = s sum_k Pp(i,k) X_k
      if (tid == 0) {
        tcgen05_fence_after();
        for (int i = 0; i < 2; ++i) {
          uint32_t acc = 0;
          for (int k = 0; k < 2; ++k)
            for (int slice = 0; slice < 2; ++slice) {
              uint32_t a_addr;
              bool a_mn;
              oc2_sym_operand(s_addr, i, k, slice, a_addr, a_mn);
              // B[n][k'] = X_k[k'][n]: MN-major over row block k's tiles, K = 64 of its rows per slice
              oc_mma_slice(tmem_base + 256 * i, a_addr, a_mn, x_addr + k * ct_n * OC_TILE_BYTES + slice * (OC_TILE_BYTES / 2),
                           true, 64 * ct_n, acc);
            }
        }
        tcgen05_commit(mma_bar);
      }
      wait_mma();   // every product that read X has completed: X may be overwritten
      if (!ok) break;
      for (int i = 0; i < 2; ++i)
        oc_drain(tmem_row, 256 * i, 2 * ct_n, x_ptr + i * ct_n * OC_TILE_BYTES, tid, first ? s : 1.0f, 0.0f, 0);
      publish();
    }
    if (!ok) break;
    oc_store_result(args, x_ptr, b, tid);
    __syncthreads();   // the tiles are free for the next block's TMA loads
  }

  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) __nanosleep(1000);   // let bulk copies already issued land
    __syncthreads();
  }
  if (warp == 0) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(static_cast<uint32_t>(OC_TMEM_COLS))
                 : "memory");
  }
}

}  // namespace tc

namespace {
// wide or square, two row blocks
bool fits_two_row_blocks(int rows, int cols) { return rows > 128 && rows <= 256 && cols >= rows && cols <= 256; }
}  // namespace

bool ns_onchip_fits(int rows, int cols) {
  if (rows % 8 != 0 || cols % 8 != 0) return false;
  const int m = rows < cols ? rows : cols, n = rows < cols ? cols : rows;
  return (m > 64 && m <= 128 && n <= 384) || fits_two_row_blocks(rows, cols);
}

int ns_onchip(const void* x, void* out, const float* inv_norm, int batch, int rows, int cols, float beta, float kappa,
              float c, void* const* upd_w, int upd_f32, float upd_alpha, int32_t* status, cudaStream_t st) {
  using namespace tc;
  MMB_REQUIRE(ns_onchip_fits(rows, cols), "on-chip Newton-Schulz: block %d x %d does not fit", rows, cols);
  MMB_REQUIRE(aligned16(x) && (out == nullptr || aligned16(out)), "on-chip Newton-Schulz needs 16-byte aligned blocks");
  OnchipArgs a;
  a.batch = batch; a.rows = rows; a.cols = cols;
  const bool two = fits_two_row_blocks(rows, cols);
  a.tall = rows > cols ? 1 : 0;
  a.row_tiles = (rows + 127) / 128;
  a.col_tiles = a.tall ? 2 : (cols + 63) / 64;        // 64 < m <= 128: the short side spans two 64-wide tiles
  a.inv_norm = inv_norm;
  a.beta = beta; a.kappa = kappa; a.c = c;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.upd_w = upd_w; a.upd_alpha = upd_alpha; a.upd_f32 = upd_f32;
  a.status = status;
  a.wait_limit = WAIT_LIMIT_CYCLES;
  CUtensorMap map;
  int rc = make_map(&map, x, batch, rows, cols, 128);
  if (rc != MMB_OK) return rc;
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "on-chip Newton-Schulz: no CUDA device");
  const int grid = batch < sms ? batch : sms;
  if (two) {
    MMB_CUDA_CHECK(cudaFuncSetAttribute(ns_onchip2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, OC2_SMEM_BYTES));
    ns_onchip2_kernel<<<grid, OC_THREADS, OC2_SMEM_BYTES, st>>>(map, a);
  } else {
    MMB_CUDA_CHECK(cudaFuncSetAttribute(ns_onchip_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, OC_SMEM_BYTES));
    ns_onchip_kernel<<<grid, OC_THREADS, OC_SMEM_BYTES, st>>>(map, a);
  }
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

}  // namespace mmb
