// Batched bf16 GEMM for Newton-Schulz on sm_100a: TMA -> shared memory ->
// tcgen05.mma -> TMEM -> shared memory -> TMA store.
//
//   D[b] = sigma_b * alpha * opA[b] . opB[b]^T + diag * I
//
// opA is M x K, opB is N x K.  Each operand has a storage mode:
//   K    stored [rows][K]  (K contiguous)
//   MN   stored [K][rows]  (rows contiguous) - used so that X^T X and P X run
//        on the matrices as stored; nothing is ever transposed in memory
//   SYM  a symmetric rows x rows matrix of which only the block-upper part is
//        stored (blocks of 256 x 256 on or above the block diagonal).  A tile
//        of the operand that lies in the stored part is fetched K-major; one
//        that lies below is fetched from its mirror image as an MN-major tile.
//        tcgen05.mma takes the major-ness per instruction, so both kinds mix
//        freely inside one K loop.
// With `sym_out` the output is such a symmetric matrix and only its block-upper
// tiles are computed (62.5 % of the tiles of a 1024 x 1024 Gram matrix), and
// nothing has to be mirrored because every consumer reads it through SYM.
//
// The epilogue needs no addend: the quintic polynomial is used in completed-
// square form, so every GEMM of the iteration is "scale, add a constant on the
// diagonal, round to bf16".
//
// CTA = 416 threads, persistent over output tiles of 128 x BN:
//   warps 0,10-12  TMA producers (two for the A tile, two for the B tile, taking
//               K slices in turn): one lane each issues cp.async.bulk.tensor
//               loads into a ring of STAGES buffers (128-byte swizzle), arming
//               the stage's mbarrier with its byte count.  Each CTA loads its own data.
//   warp 1      MMA issuer: one lane issues four tcgen05.mma (K=16 each) per
//               stage into one of two TMEM accumulators (128 lanes x BN fp32
//               columns each); tcgen05.commit frees the stage, and after the
//               last K slice hands the accumulator to the epilogue.
//   warps 2-9   epilogue: each warp takes 32 rows x 64 columns at a time
//               (tcgen05.ld), scales, adds the diagonal, rounds to bf16, writes a
//               swizzled piece into its own 4 KiB staging buffer and issues its
//               own TMA store - no barrier couples the epilogue warps.  The
//               second accumulator lets this overlap the next tile's main loop;
//               TMA clips rows/columns beyond M/N, so ragged edges need no masks.
//
// PAIR variant (used when M > 128 and N > 128): two CTAs of a cluster share one
// 256 x 256 tile through tcgen05.mma cta_group::2.  Each CTA loads 128 rows of A
// and 128 rows of B per K slice (32 KiB instead of 48 KiB per SM and K slice,
// so a third less operand traffic from L2, and six stages instead of four);
// the even CTA issues the MMAs for both, each CTA drains its own 128 x 256 half
// of the accumulator.  Loads are plain per-CTA TMA loads (cta_group::2 only so
// that the peer's loads can signal the issuing CTA's barrier); each CTA
// fetches its own operands, nothing is broadcast across the cluster.
//
// Every mbarrier wait is bounded (about two seconds of wall clock): on expiry
// the waiting role stores a code in the device status word, raises a CTA-wide
// abort flag and all roles leave their loops; the CTA then lets outstanding
// bulk copies land, frees its TMEM and returns.  Nothing traps.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "gemm.cuh"
#include "tcgen05_ptx.cuh"

namespace mmb {
namespace tc {


constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_EPI_WARPS = 8;
constexpr int PRODUCERS_PER_OPERAND = 2;         // producer warps per operand, taking K slices in turn
constexpr int FIRST_EXTRA_PRODUCER = 2 + NUM_EPI_WARPS;  // warp 0 is a producer too
constexpr int NUM_THREADS = 32 * (2 + NUM_EPI_WARPS + 2 * PRODUCERS_PER_OPERAND - 1);
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int CHUNK_BYTES = 64 * BK * 2;      // one 64-wide MN-major chunk (8 KiB)
constexpr int EPI_WARP_BYTES = 32 * 64 * 2;   // one epilogue warp's staging buffer: 32 rows x 64 columns of bf16
constexpr int EPI_BYTES = NUM_EPI_WARPS * EPI_WARP_BYTES;
constexpr int SYM_SHIFT = 8;                  // symmetric storage granularity: 256
constexpr int SCHED_DEPTH = 4;                // tile numbers a pair may hold ahead of its consumers (dynamic schedule)
constexpr int SCHED_CONSUMERS_PER_CTA = 2 * PRODUCERS_PER_OPERAND + NUM_EPI_WARPS;  // plus the MMA thread in the even CTA

template <int BN, bool PAIR>
struct Cfg {
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;  // rows of B this CTA stages
  static constexpr int B_TILE_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
  static constexpr int STAGES = PAIR ? 6 : (BN == 256 ? 4 : (BN == 128 ? 6 : 7));
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;   // rows of the output tile (both CTAs of a pair)
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

struct GemmArgs {
  int M, N, K, batch;
  int tiles_m, tiles_n, tiles_per_batch;
  long long total_tiles;
  int a_mode, b_mode, sym_out;
  float alpha, diag;
  const float* inv_norm;
  int sigma_pow;
  int32_t* status;
  int* sched;  // dynamic schedule: [0] next tile number, [1] pairs that have seen the end; both 0 at launch
  // fused weight update (UPD kernels): the result is not stored; instead W[b] <- W[b] + upd_alpha * bf16(result)
  void* const* upd_w;   // per batch entry, pointer to that block's M x N weights (row-major, 16-byte aligned)
  float upd_alpha;
  int upd_f32;          // weights are fp32 (else bf16)
  long long wait_limit; // SM cycles a role may wait on a barrier before it gives up
  int pdl;              // launched with programmatic stream serialisation: wait for the previous kernel here
};

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle (built in the MMA issue loop):
//   bits  0-13  start address >> 4
//   bits 16-29  leading-dimension byte offset >> 4
//   bits 32-45  stride-dimension byte offset >> 4
//   bits 46-47  descriptor version (1 on sm_100)
//   bits 61-63  swizzle mode (2 = 128 bytes)
// K-major tile ([rows][64] bf16, 128 bytes per row): 8-row groups are 1024
// bytes apart (stride offset); the leading offset is unused (1).
// MN-major tile ([64 k][64 rows] chunks of 8 KiB): the 8-k groups of one
// chunk are 1024 bytes apart (stride offset) and the 64-row chunks are 8 KiB
// apart (leading offset).
//
// Instruction descriptor, kind::f16: fp32 accumulate, bf16 A and B.
//   bits 4-5 D format (1 = f32); 7-9 A format (1 = bf16); 10-12 B format;
//   bit 15 / 16: A / B is MN-major; bits 17-22 N>>3; bits 24-28 M>>4.

// Is the operand tile with first row r0 and first k k0 fetched K-major?
__device__ __forceinline__ bool fetch_kmajor(int mode, int r0, int k0) {
  return mode == GEMM_K || (mode == GEMM_SYM && (r0 >> SYM_SHIFT) <= (k0 >> SYM_SHIFT));
}

// Tile t of the launch -> batch, first row, first column.  Tiles are TILE_M rows
// by BN columns.  With sym_out only tiles with (n0 >> 8) >= (m0 >> 8) exist:
// the tile rows of 256-block p own the column tiles p .. tiles_n-1.
template <int BN, int TILE_M>
__device__ __forceinline__ void tile_coords(long long t, const GemmArgs& a, int& b, int& m0, int& n0) {
  b = static_cast<int>(t / a.tiles_per_batch);
  int r = static_cast<int>(t - static_cast<long long>(b) * a.tiles_per_batch);
  if (a.sym_out && BN == 256) {
    constexpr int ROWS_PER_BLOCK = 256 / TILE_M;  // tile rows per 256-block: 2 (single CTA) or 1 (pair)
    int p = 0;
    for (;; ++p) {
      const int rows = (a.tiles_m - ROWS_PER_BLOCK * p) >= ROWS_PER_BLOCK ? ROWS_PER_BLOCK : 1;
      const int cnt = rows * (a.tiles_n - p);
      if (r < cnt) break;
      r -= cnt;
    }
    const int w = a.tiles_n - p;
    const int hi = r >= w ? 1 : 0;
    m0 = (ROWS_PER_BLOCK * p + hi) * TILE_M;
    n0 = (p + r - hi * w) * BN;
  } else {
    m0 = (r / a.tiles_n) * TILE_M;
    n0 = (r % a.tiles_n) * BN;
  }
}

// Dynamic schedule (pairs only).  Lane 0 of warp 1 of the odd CTA - idle otherwise - draws tile numbers
// from a global counter and publishes each into a ring of SCHED_DEPTH slots in both CTAs' shared memory
// (own slot: plain store + arrive; peer's slot: st.shared::cluster + arrive.release.cluster).  Every
// consumer (4 producer lanes and 8 epilogue warps per CTA, the MMA lane of the even CTA) walks the ring
// with its own cursor and returns each slot by arriving at the odd CTA's `sched_empty` barrier.  A pair
// that starts late or shares its SMs with another kernel simply draws fewer tiles.  -1 ends the walk.
struct TileCursor {
  uint32_t n = 0;  // tiles drawn so far by this consumer
};
__device__ __forceinline__ long long draw_tile(TileCursor& c, uint32_t sched_full, uint32_t sched_empty,
                                               const volatile int* slots, volatile int* abort_flag, int32_t* status,
                                               long long limit) {
  const uint32_t q = c.n % SCHED_DEPTH, ph = (c.n / SCHED_DEPTH) & 1u;
  if (!mbar_wait<true>(sched_full + 8 * q, ph, abort_flag, status, STATUS_WAIT_SCHED_FULL, limit)) return -1;
  const int t = slots[q];
  mbar_arrive_cluster(mapa(sched_empty + 8 * q, 1));   // the ring's owner is the odd CTA (also when that is us)
  ++c.n;
  return t;
}

// -------------------------------------------------------------------- kernel
// 112 registers per thread (13 warps: 46,592 of the SM's 65,536) leave room for one 256-thread CTA of a
// streaming kernel (64 registers) on the same SM, so momentum / update / AdamW launches on another
// stream run beside the GEMMs instead of queueing behind them.
// UPD: the epilogue does not store the result; it rounds it to bf16 (the value the plain epilogue would
// have stored) and applies the Muon weight update W <- W + alpha * result to the block's weights in place,
// with one fused multiply-add and one rounding to the weights' type (what torch's add_(other, alpha=) does).
template <int BN, bool PAIR, bool DYN = false, bool UPD = false>
__global__ void __maxnreg__(112)
gemm_kernel(const __grid_constant__ CUtensorMap map_a_k, const __grid_constant__ CUtensorMap map_a_mn,
            const __grid_constant__ CUtensorMap map_b_k, const __grid_constant__ CUtensorMap map_b_mn,
            const __grid_constant__ CUtensorMap map_d, const GemmArgs args) {
  using C = Cfg<BN, PAIR>;
  constexpr int STAGES = C::STAGES;
  constexpr int TILE_M = C::TILE_M;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw_addr + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw_addr);
  const uint32_t epi_addr = tiles_addr + STAGES * C::STAGE_BYTES;  // one 4 KiB staging buffer per epilogue warp
  uint8_t* epi_ptr = tiles_ptr + STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_ptr + EPI_BYTES);
  const uint32_t bars_addr = epi_addr + EPI_BYTES;
  const uint32_t full_bar = bars_addr;                      // STAGES (pair: only the even CTA's are used)
  const uint32_t empty_bar = bars_addr + 8 * STAGES;        // STAGES
  const uint32_t tmem_full_bar = bars_addr + 16 * STAGES;   // 2
  const uint32_t tmem_empty_bar = tmem_full_bar + 16;       // 2 (pair: only the even CTA's are used)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // dynamic schedule: two rings of barriers and the slots, behind the words above
  const uint32_t sched_full = bars_addr + 8 * (2 * STAGES + 4) + 16;
  const uint32_t sched_empty = sched_full + 8 * SCHED_DEPTH;
  volatile int* sched_slots = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 4 + 2 + 2 * SCHED_DEPTH);
  static_assert(!DYN || PAIR, "the dynamic schedule is built on the idle warp of a pair's odd CTA");
  static_assert(8 * (2 * STAGES + 4) + 16 + 16 * SCHED_DEPTH + 4 * SCHED_DEPTH <= 256, "barrier area overflow");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k_tiles = (args.K + BK - 1) / BK;
  // In a pair the even CTA of the cluster issues the MMAs; each CTA owns rows
  // [128*cta_rank, +128) of the tile for A and for the output, and the same
  // rows of the B tile.
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const long long first_tile = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const long long tile_step = PAIR ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar + 8 * s, PAIR ? 4 : 2);  // one expect-tx arrival per producer warp (of both CTAs)
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full_bar + 8 * i, 1);
      mbar_init(tmem_empty_bar + 8 * i, (PAIR ? 2 : 1) * NUM_EPI_WARPS);  // one arrival per epilogue warp (of both CTAs)
    }
    if (DYN) {
      for (int i = 0; i < SCHED_DEPTH; ++i) {
        mbar_init(sched_full + 8 * i, 1);
        mbar_init(sched_empty + 8 * i, 2 * SCHED_CONSUMERS_PER_CTA + 1);
      }
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(static_cast<uint32_t>(C::TMEM_COLS))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(static_cast<uint32_t>(C::TMEM_COLS))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync();  // the peer's barriers exist before anything is signalled across
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (args.pdl) {
    // Everything above touched only this CTA's shared and tensor memory, so it may run while the previous
    // kernel of the stream is still finishing.  From here on global memory is read and written.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  if (warp == 0 || warp >= FIRST_EXTRA_PRODUCER) {
    // ------------------------------------------------------ TMA producers
    // Issuing a bulk tensor copy keeps the issuing thread busy for several hundred cycles, so one
    // thread cannot feed a 64-deep K slice per 512 cycles of MMA work.  2 x PRODUCERS_PER_OPERAND warps
    // share the job: producer p of an operand loads that operand's tile for the K slices whose running
    // number is congruent to p, and arms the stage's barrier with its own byte count.
    const int pid = warp == 0 ? 0 : warp - FIRST_EXTRA_PRODUCER + 1;  // 0 .. 2*PRODUCERS_PER_OPERAND-1
    const bool is_a = (pid & 1) == 0;
    const uint32_t turn = static_cast<uint32_t>(pid >> 1);
    if (lane == 0) {
      uint32_t slice = 0;  // running number of the K slice over all tiles of this CTA
      bool ok = true;
      const int mode = is_a ? args.a_mode : args.b_mode;
      const int chunks = is_a ? BM / 64 : C::B_ROWS / 64;
      const uint32_t bytes = is_a ? A_TILE_BYTES : C::B_TILE_BYTES;
      const CUtensorMap* map_k = is_a ? &map_a_k : &map_b_k;
      const CUtensorMap* map_mn = is_a ? &map_a_mn : &map_b_mn;
      TileCursor cursor;
      for (long long t = DYN ? draw_tile(cursor, sched_full, sched_empty, sched_slots, abort_flag, args.status, args.wait_limit) : first_tile;
           ok && t >= 0 && t < args.total_tiles;
           t = DYN ? draw_tile(cursor, sched_full, sched_empty, sched_slots, abort_flag, args.status, args.wait_limit) : t + tile_step) {
        int b, m0, n0;
        tile_coords<BN, TILE_M>(t, args, b, m0, n0);
        const int r_tile = is_a ? m0 : n0;                       // decides K-major vs mirrored fetch
        const int r_cta = is_a ? m0 + static_cast<int>(cta_rank) * BM : n0 + static_cast<int>(cta_rank) * C::B_ROWS;
        for (int kt = 0; kt < num_k_tiles; ++kt, ++slice) {
          if (slice % PRODUCERS_PER_OPERAND != turn) continue;
          const uint32_t stage = slice % STAGES;
          const uint32_t phase = (slice / STAGES) & 1u;
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, args.status, STATUS_WAIT_PRODUCER_EMPTY, args.wait_limit)) {
            ok = false;
            break;
          }
          const uint32_t dst = tiles_addr + stage * C::STAGE_BYTES + (is_a ? 0 : A_TILE_BYTES);
          const int k0 = kt * BK;
          const bool kmajor = fetch_kmajor(mode, r_tile, k0);
          if (PAIR) {
            const uint32_t fb = mapa(full_bar + 8 * stage, 0);  // the even CTA's barrier
            mbar_expect_tx_cluster(fb, bytes);
            if (kmajor) {
              tma_load_3d_pair(dst, map_k, fb, k0, r_cta, b);
            } else {
              for (int c = 0; c < chunks; ++c) tma_load_3d_pair(dst + c * CHUNK_BYTES, map_mn, fb, r_cta + 64 * c, k0, b);
            }
          } else {
            const uint32_t fb = full_bar + 8 * stage;
            mbar_expect_tx(fb, bytes);
            if (kmajor) {
              tma_load_3d(dst, map_k, fb, k0, r_cta, b);
            } else {
              for (int c = 0; c < chunks; ++c) tma_load_3d(dst + c * CHUNK_BYTES, map_mn, fb, r_cta + 64 * c, k0, b);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------------------- MMA issuer
    // One thread issues everything; each tcgen05.mma costs it on the order of a hundred cycles, so the
    // loop body is kept to the wait, four MMAs and the commit.
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t K_STEP = (UMMA_K * 2) >> 4;     // K-major: 32 bytes per K=16, in 16-byte units
      constexpr uint32_t MN_STEP = (UMMA_K * 128) >> 4;  // MN-major: 16 rows of 128 bytes
      constexpr uint32_t LBO_MN = CHUNK_BYTES >> 4;
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);  // bits 32-63 of the descriptor
      constexpr uint32_t IDESC_BASE = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                      (static_cast<uint32_t>(TILE_M >> 4) << 24);
      const bool a_fixed = args.a_mode != GEMM_SYM, b_fixed = args.b_mode != GEMM_SYM;
      uint32_t stage = 0, phase = 0;
      uint32_t local = 0;
      bool ok = true;
      TileCursor cursor;
      for (long long t = DYN ? draw_tile(cursor, sched_full, sched_empty, sched_slots, abort_flag, args.status, args.wait_limit) : first_tile;
           ok && t >= 0 && t < args.total_tiles;
           t = DYN ? draw_tile(cursor, sched_full, sched_empty, sched_slots, abort_flag, args.status, args.wait_limit) : t + tile_step, ++local) {
        int b, m0, n0;
        tile_coords<BN, TILE_M>(t, args, b, m0, n0);
        const uint32_t acc = local & 1u;
        const uint32_t acc_phase = (local >> 1) & 1u;
        if (!mbar_wait(tmem_empty_bar + 8 * acc, acc_phase ^ 1u, abort_flag, args.status, STATUS_WAIT_MMA_TMEM_EMPTY, args.wait_limit)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();  // the epilogue's reads of this accumulator are ordered before the overwrite
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ak = args.a_mode == GEMM_K, bk = args.b_mode == GEMM_K;
        uint32_t accumulate = 0;
        for (int kt = 0; kt < num_k_tiles; ++kt) {
          if (!a_fixed) ak = fetch_kmajor(GEMM_SYM, m0, kt * BK);
          if (!b_fixed) bk = fetch_kmajor(GEMM_SYM, n0, kt * BK);
          // descriptor halves: high = stride offset | version | swizzle, low = address | leading offset
          const uint32_t sa = (tiles_addr + stage * C::STAGE_BYTES) >> 4;
          const uint32_t a_lo = sa | ((ak ? 1u : LBO_MN) << 16);
          const uint32_t b_lo = (sa + (A_TILE_BYTES >> 4)) | ((bk ? 1u : LBO_MN) << 16);
          const uint32_t idesc = IDESC_BASE | ((ak ? 0u : 1u) << 15) | ((bk ? 0u : 1u) << 16);
          const uint32_t a_step = ak ? K_STEP : MN_STEP;
          const uint32_t b_step = bk ? K_STEP : MN_STEP;
          if (!mbar_wait(full_bar + 8 * stage, phase, abort_flag, args.status, STATUS_WAIT_MMA_FULL, args.wait_limit)) {
            ok = false;
            break;
          }
          tcgen05_mma_f16_split<PAIR>(d_tmem, a_lo, DESC_HI, b_lo, DESC_HI, idesc, accumulate);
#pragma unroll
          for (uint32_t k = 1; k < BK / UMMA_K; ++k)
            tcgen05_mma_f16_split<PAIR>(d_tmem, a_lo + k * a_step, DESC_HI, b_lo + k * b_step, DESC_HI, idesc, 1u);
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if (PAIR) tcgen05_commit_pair(empty_bar + 8 * stage); else tcgen05_commit(empty_bar + 8 * stage);
          accumulate = 1u;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {  // accumulator complete
          if (PAIR) tcgen05_commit_pair(tmem_full_bar + 8 * acc); else tcgen05_commit(tmem_full_bar + 8 * acc);
        }
      }
    } else if (DYN && lane == 0 && cta_rank == 1) {
      // ------------------------------------------------------ tile scheduler
      const int total = static_cast<int>(args.total_tiles);
      for (uint32_t i = 0;; ++i) {
        const uint32_t q = i % SCHED_DEPTH, ph = (i / SCHED_DEPTH) & 1u;
        // every consumer of both CTAs has read the slot's previous tile (immediate on the first lap)
        if (!mbar_wait<true>(sched_empty + 8 * q, ph ^ 1u, abort_flag, args.status, STATUS_WAIT_SCHED_EMPTY, args.wait_limit)) break;
        const int drawn = atomicAdd(args.sched, 1);
        const int tile = drawn < total ? drawn : -1;
        sched_slots[q] = tile;
        st_shared_cluster_s32(mapa(smem_u32(const_cast<int*>(sched_slots + q)), 0), tile);
        mbar_arrive(sched_full + 8 * q);
        mbar_arrive_cluster(mapa(sched_full + 8 * q, 0));
        if (tile < 0) {
          // The pair that sees the end last (no draw can follow it) rearms the counters for the next launch.
          const int pairs = static_cast<int>(gridDim.x >> 1);
          if (atomicAdd(args.sched + 1, 1) == pairs - 1) {
            args.sched[0] = 0;
            args.sched[1] = 0;
            __threadfence();
          }
          break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    // Eight warps: warp w may touch TMEM lanes [32*(w%4), +32) only, so two warps share each quarter of
    // the rows and split the 64-column chunks between them (even / odd).  Every warp works alone: it
    // stages its 32 x 64 piece in its own buffer and issues its own TMA store, so no barrier couples
    // the warps and a store's latency is hidden behind the other warps' work.
    const int ew = warp - 2;
    const int quarter = warp & 3;
    const int half = ew >> 2;
    uint8_t* my_buf = epi_ptr + ew * EPI_WARP_BYTES;
    const uint32_t my_buf_addr = epi_addr + ew * EPI_WARP_BYTES;
    uint32_t local = 0;
    bool ok = true;
    TileCursor cursor;
    auto next_tile = [&](long long prev) -> long long {
      if (!DYN) return prev < 0 ? first_tile : prev + tile_step;
      long long t = 0;
      if (lane == 0) t = draw_tile(cursor, sched_full, sched_empty, sched_slots, abort_flag, args.status, args.wait_limit);
      return __shfl_sync(0xffffffffu, t, 0);
    };
    for (long long t = next_tile(-1); ok && t >= 0 && t < args.total_tiles; t = next_tile(t), ++local) {
      int b, m0, n0;
      tile_coords<BN, TILE_M>(t, args, b, m0, n0);
      m0 += static_cast<int>(cta_rank) * BM;  // this CTA's half of a pair tile
      const uint32_t acc = local & 1u;
      const uint32_t acc_phase = (local >> 1) & 1u;
      uint8_t* w_base = nullptr;  // UPD: this block's weights
      if (UPD) {
        w_base = static_cast<uint8_t*>(args.upd_w[b]);
        // pull this warp's pieces of W towards L2 while the accumulator is still being computed: lane = row
        const int wrow = m0 + quarter * 32 + lane;
        if (wrow < args.M) {
          const int esz = args.upd_f32 ? 4 : 2;
          const uint8_t* w_row = w_base + static_cast<long long>(wrow) * args.N * esz;
          for (int c = half; c < BN / 64; c += 2) {
            const int col0 = n0 + c * 64;
            if (col0 >= args.N) break;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(w_row + static_cast<long long>(col0) * esz));
            if (args.upd_f32 && col0 + 32 < args.N)
              asm volatile("prefetch.global.L2 [%0];" ::"l"(w_row + static_cast<long long>(col0 + 32) * esz));
          }
        }
      }
      if (!mbar_wait(tmem_full_bar + 8 * acc, acc_phase, abort_flag, args.status, STATUS_WAIT_EPI_TMEM_FULL, args.wait_limit)) {
        ok = false;
        break;
      }
      tcgen05_fence_after();
      float sigma = 1.0f;
      if (args.sigma_pow > 0) {
        const float s = args.inv_norm[b];
        sigma = args.sigma_pow == 2 ? s * s : s;
      }
      const float scale = sigma * args.alpha;
      const int row0 = m0 + quarter * 32;  // first row of this warp's piece
      const int row = row0 + lane;
      const uint32_t t_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = half; c < BN / 64; c += 2) {
        const int col0 = n0 + c * 64;
        if (col0 >= args.N || row0 >= args.M) break;  // uniform across the warp
        uint32_t v[64];
        tcgen05_ld_32x32b_x32(t_base + c * 64, v);
        tcgen05_ld_32x32b_x32(t_base + c * 64 + 32, v + 32);
        tcgen05_wait_ld();
        const int dcol = row - col0;  // column of this row's diagonal element inside the chunk, if any
        uint4 ov[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov[q]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e = 8 * q + 2 * i;
            float x0 = scale * __uint_as_float(v[e]);
            float x1 = scale * __uint_as_float(v[e + 1]);
            if (e == dcol) x0 += args.diag;
            if (e + 1 == dcol) x1 += args.diag;
            oh[i] = __floats2bfloat162_rn(x0, x1);
          }
        }
        if (!UPD && lane == 0) bulk_wait_read_0();  // this warp's previous store has left the buffer
        __syncwarp();
        // 128-byte swizzle: 16-byte unit q of row r lives at unit q ^ (r & 7)
        uint8_t* rowp = my_buf + lane * 128;
#pragma unroll
        for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(rowp + ((q ^ (lane & 7)) << 4)) = ov[q];
        if (!UPD) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&map_d, my_buf_addr, col0, row0, b);
            bulk_commit();
          }
        } else {
          // The piece (32 rows x 64 columns of bf16, the value the plain epilogue stores) is read back row
          // by row so that the weights are touched in whole 128-byte lines: eight lanes per row, four rows
          // per pass.  W <- fma(alpha, piece, W), one rounding to the weights' type.
          __syncwarp();
          const int q = lane & 7;
          const int col = col0 + 8 * q;
          uint4 pv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            pv[i] = *reinterpret_cast<const uint4*>(my_buf + r * 128 + ((q ^ (r & 7)) << 4));
          }
          __syncwarp();                                  // the buffer may be overwritten by the next chunk
          if (col < args.N) {
            if (args.upd_f32) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int grow = row0 + 4 * i + (lane >> 3);
                if (grow >= args.M) break;
                float4* wp = reinterpret_cast<float4*>(w_base + (static_cast<long long>(grow) * args.N + col) * 4);
                float4 w0 = __ldcs(wp), w1 = __ldcs(wp + 1);
                const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&pv[i]);
                const float2 o0 = __bfloat1622float2(oh[0]), o1 = __bfloat1622float2(oh[1]);
                const float2 o2 = __bfloat1622float2(oh[2]), o3 = __bfloat1622float2(oh[3]);
                w0.x = fmaf(args.upd_alpha, o0.x, w0.x); w0.y = fmaf(args.upd_alpha, o0.y, w0.y);
                w0.z = fmaf(args.upd_alpha, o1.x, w0.z); w0.w = fmaf(args.upd_alpha, o1.y, w0.w);
                w1.x = fmaf(args.upd_alpha, o2.x, w1.x); w1.y = fmaf(args.upd_alpha, o2.y, w1.y);
                w1.z = fmaf(args.upd_alpha, o3.x, w1.z); w1.w = fmaf(args.upd_alpha, o3.y, w1.w);
                __stcs(wp, w0);
                __stcs(wp + 1, w1);
              }
            } else {
              uint4 wv[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {              // all eight loads in flight before the first use
                const int grow = row0 + 4 * i + (lane >> 3);
                if (grow < args.M)
                  wv[i] = __ldcs(reinterpret_cast<const uint4*>(w_base + (static_cast<long long>(grow) * args.N + col) * 2));
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int grow = row0 + 4 * i + (lane >> 3);
                if (grow >= args.M) break;
                const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&pv[i]);
                __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&wv[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 o = __bfloat1622float2(oh[j]);
                  const float2 w = __bfloat1622float2(wh[j]);
                  wh[j] = __floats2bfloat162_rn(fmaf(args.upd_alpha, o.x, w.x), fmaf(args.upd_alpha, o.y, w.y));
                }
                __stcs(reinterpret_cast<uint4*>(w_base + (static_cast<long long>(grow) * args.N + col) * 2), wv[i]);
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa(tmem_empty_bar + 8 * acc, 0)); else mbar_arrive(tmem_empty_bar + 8 * acc);
      }
    }
    if (!UPD && lane == 0) bulk_wait_all();
  }

  // ------------------------------------------------------------- teardown
  __syncthreads();
  if (*abort_flag) {
    // let bulk copies that were already issued land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) __nanosleep(1000);  // about 200 microseconds
    __syncthreads();
  }
  if (PAIR) cluster_sync();  // neither CTA leaves (or frees TMEM) while its peer may still signal or write to it
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(static_cast<uint32_t>(C::TMEM_COLS))
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(static_cast<uint32_t>(C::TMEM_COLS))
                   : "memory");
  }
}

// ---------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map over a bf16 array [batch][outer][inner] (inner contiguous) with a
// box of {64, box_outer, 1} and 128-byte swizzle; out-of-range elements read 0
// and are not written.
int make_map(CUtensorMap* map, const void* base, int batch, int outer, int inner, int box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(MMB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(inner) * 2ull, static_cast<cuuint64_t>(inner) * outer * 2ull};
  cuuint32_t box[3] = {64u, static_cast<cuuint32_t>(box_outer), 1u};
  cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MMB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for [%d][%d][%d] box %d", static_cast<int>(r), batch,
                outer, inner, box_outer);
  return MMB_OK;
}

// Maps of one operand: K-major view (box rows x 64 k) and MN-major view (64 k x 64 rows).
int operand_maps(CUtensorMap* k_map, CUtensorMap* mn_map, const void* base, int batch, int rows, int K, int mode,
                 int box_rows) {
  int rc;
  if (mode == GEMM_K) {
    if ((rc = make_map(k_map, base, batch, rows, K, box_rows)) != MMB_OK) return rc;
    *mn_map = *k_map;  // never used
  } else if (mode == GEMM_MN) {
    if ((rc = make_map(mn_map, base, batch, K, rows, BK)) != MMB_OK) return rc;
    *k_map = *mn_map;  // never used
  } else {
    if ((rc = make_map(k_map, base, batch, rows, K, box_rows)) != MMB_OK) return rc;
    if ((rc = make_map(mn_map, base, batch, K, rows, BK)) != MMB_OK) return rc;
  }
  return MMB_OK;
}

template <int BN, bool PAIR, bool DYN = false, bool UPD = false>
int launch(const CUtensorMap* maps, const GemmArgs& args, int grid, cudaStream_t st) {
  auto kern = gemm_kernel<BN, PAIR, DYN, UPD>;
  constexpr int smem = Cfg<BN, PAIR>::SMEM_BYTES;
  MMB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = args.pdl ? 2 : 1;
  MMB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[2], maps[3], maps[4], args));
  count_launch();
  return MMB_OK;
}

}  // namespace tc

// How many CTAs (single) or clusters (pair) of the 256-wide kernel the device can hold at once.
int gemm_occupancy(int pair, int* out) {
  using namespace tc;
  cudaLaunchConfig_t cfg = {};
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "mmb_gemm_occupancy: no CUDA device");
  cfg.gridDim = dim3(pair ? 2 * (sms / 2) : sms, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (pair) {
    cfg.dynamicSmemBytes = Cfg<256, true>::SMEM_BYTES;
    MMB_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg<256, true>::SMEM_BYTES));
    MMB_CUDA_CHECK(cudaOccupancyMaxActiveClusters(out, gemm_kernel<256, true>, &cfg));
  } else {
    cfg.dynamicSmemBytes = Cfg<256, false>::SMEM_BYTES;
    MMB_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg<256, false>::SMEM_BYTES));
    MMB_CUDA_CHECK(cudaOccupancyMaxActiveClusters(out, gemm_kernel<256, false>, &cfg));
  }
  return MMB_OK;
}

int gemm_tcgen05(const GemmCall& g, int32_t* status, cudaStream_t st) {
  using namespace tc;
  MMB_REQUIRE(g.M % 8 == 0 && g.N % 8 == 0 && g.K % 8 == 0, "tcgen05 GEMM needs M, N, K multiples of 8 (got %d %d %d)",
              g.M, g.N, g.K);
  MMB_REQUIRE(aligned16(g.a) && aligned16(g.b) && aligned16(g.d), "tcgen05 GEMM needs 16-byte aligned operands");
  if (g.a_mode == GEMM_SYM) MMB_REQUIRE(g.M == g.K, "symmetric A operand must be square (M == K)");
  if (g.b_mode == GEMM_SYM) MMB_REQUIRE(g.N == g.K, "symmetric B operand must be square (N == K)");
  if (g.sym_out) MMB_REQUIRE(g.M == g.N, "symmetric output must be square");
  const int bn = g.N > 128 ? 256 : (g.N > 64 ? 128 : 64);
  // two CTAs per 256 x 256 tile when the problem has at least two tile rows of 128
  const bool pair = bn == 256 && g.M > BM;
  const int tile_m = pair ? 2 * BM : BM;
  CUtensorMap maps[5];
  int rc;
  if ((rc = operand_maps(&maps[0], &maps[1], g.a, g.batch, g.M, g.K, g.a_mode, BM)) != MMB_OK) return rc;
  if ((rc = operand_maps(&maps[2], &maps[3], g.b, g.batch, g.N, g.K, g.b_mode, pair ? bn / 2 : bn)) != MMB_OK) return rc;
  if ((rc = make_map(&maps[4], g.d, g.batch, g.M, g.N, 32)) != MMB_OK) return rc;  // one epilogue warp's piece
  GemmArgs args;
  args.M = g.M; args.N = g.N; args.K = g.K; args.batch = g.batch;
  args.tiles_m = (g.M + tile_m - 1) / tile_m;
  args.tiles_n = (g.N + bn - 1) / bn;
  args.sym_out = (g.sym_out && bn == 256) ? 1 : 0;
  if (args.sym_out) {
    const int rows_per_block = 256 / tile_m;
    int cnt = 0;
    for (int p = 0; rows_per_block * p < args.tiles_m; ++p)
      cnt += ((args.tiles_m - rows_per_block * p) >= rows_per_block ? rows_per_block : 1) * (args.tiles_n - p);
    args.tiles_per_batch = cnt;
  } else {
    args.tiles_per_batch = args.tiles_m * args.tiles_n;
  }
  args.total_tiles = static_cast<long long>(g.batch) * args.tiles_per_batch;
  args.a_mode = g.a_mode; args.b_mode = g.b_mode;
  args.alpha = g.alpha; args.diag = g.diag;
  args.inv_norm = g.inv_norm; args.sigma_pow = g.inv_norm != nullptr ? g.sigma_pow : 0;
  args.status = status;
  args.sched = nullptr;
  args.upd_w = g.upd_w;
  args.upd_alpha = g.upd_alpha;
  args.upd_f32 = g.upd_f32;
  args.wait_limit = WAIT_LIMIT_CYCLES;
  args.pdl = gemm_dependent_launch() ? 1 : 0;
  const bool upd = g.upd_w != nullptr;
  if (upd) MMB_REQUIRE(!g.sym_out, "the fused weight update applies to a full (non-symmetric) result");
  const int sms = sm_count();
  if (sms <= 0) return fail(MMB_ERR_CUDA, "tcgen05 GEMM: no CUDA device");
  if (args.total_tiles == 0) return MMB_OK;
  if (pair) {
    const long long pairs = sms / 2;
    const int grid = 2 * static_cast<int>(args.total_tiles < pairs ? args.total_tiles : pairs);
    if (g.sched != nullptr && gemm_schedule_dynamic() && args.total_tiles < (1ll << 30)) {
      args.sched = g.sched;
      return upd ? launch<256, true, true, true>(maps, args, grid, st) : launch<256, true, true>(maps, args, grid, st);
    }
    return upd ? launch<256, true, false, true>(maps, args, grid, st) : launch<256, true>(maps, args, grid, st);
  }
  const int grid = static_cast<int>(args.total_tiles < sms ? args.total_tiles : sms);
  if (bn == 256) return upd ? launch<256, false, false, true>(maps, args, grid, st) : launch<256, false>(maps, args, grid, st);
  if (bn == 128) return upd ? launch<128, false, false, true>(maps, args, grid, st) : launch<128, false>(maps, args, grid, st);
  return upd ? launch<64, false, false, true>(maps, args, grid, st) : launch<64, false>(maps, args, grid, st);
}

// ------------------------------------------------------------ wait probe
// One warp waits, with the GEMM's own bounded wait and a caller-chosen limit, on a barrier that nothing
// ever arrives at.  The wait must expire, store its code in the status word and let the kernel return: the
// behaviour every role of the GEMM relies on when a hand-off never comes.
__global__ void wait_probe_kernel(long long limit_cycles, int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(tc::smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0)
    tc::mbar_wait(tc::smem_u32(&bar), 0, &abort_flag, status, STATUS_WAIT_PROBE, limit_cycles);
  __syncthreads();
}

int wait_probe(long long limit_cycles, int32_t* status, cudaStream_t st) {
  MMB_REQUIRE(status != nullptr, "mmb_wait_probe: null status word");
  MMB_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000ll, "mmb_wait_probe: limit of %lld cycles is outside 1..2e9",
              limit_cycles);
  wait_probe_kernel<<<1, 32, 0, st>>>(limit_cycles, status);
  MMB_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return MMB_OK;
}

}  // namespace mmb
