/*
 * monarch_muon_b200.h - C ABI of libmonarch_muon_b200.so
 *
 * The hot path of the Monarch-Muon optimizer step for NVIDIA B200 (sm_100a):
 * heavy-ball momentum with FP8 (E4M3, groups of 128) optimizer state, batched
 * quintic Newton-Schulz on bf16 blocks (tcgen05 tensor cores, TMEM, TMA), the
 * Muon weight update and the embedded AdamW.
 *
 * Conventions
 *   - Every pointer named *_dev or documented "device" is a CUDA device
 *     pointer on the current device; tables (`const mmb_*_seg*`) are HOST
 *     arrays that the call copies into kernel parameters.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default
 *     stream).  Calls only enqueue work; none synchronises the device.
 *   - Return value 0 = success.  Negative = error; mmb_last_error() returns a
 *     description (thread local).  Nothing throws, aborts or exits.
 *   - The caller owns all memory.  The library allocates nothing on the
 *     device except inside mmb_device_status_create().
 *   - Citations name the reference file (path within the reference project)
 *     and lines whose behaviour the entry point replaces.
 */
#ifndef MONARCH_MUON_B200_H
#define MONARCH_MUON_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MMB_OK 0
#define MMB_ERR_INVALID (-1) /* bad argument                                 */
#define MMB_ERR_CUDA (-2)    /* a CUDA runtime/driver call failed            */
#define MMB_ERR_DEVICE (-3)  /* a kernel reported a problem (status word)    */
#define MMB_ERR_UNSUPPORTED (-4)

/* element types */
#define MMB_BF16 0
#define MMB_F32 1

/* momentum state formats */
#define MMB_STATE_FP8_ABSMAX 0 /* E4M3 codes + one fp32 scale per 128          */
#define MMB_STATE_FP8_EXPAND 1 /* E4M3 codes + scale, expand, sqrt_minmax      */
#define MMB_STATE_BF16 2       /* plain buffer, two roundings per step         */
#define MMB_STATE_F32 3

/* Arithmetic of the FP8 quantisers.
 *   MMB_DIV_FULL  (what the Python layer passes by default) the GPU instructions the reference's Triton
 *                 kernels compile to: div.full.f32 for `/`, sqrt.approx.ftz.f32, library powf / log2f.  The
 *                 absmax codec then equals the reference's kernel bit for bit on the same GPU; the
 *                 range-expansion codec equals it in expand_ and sqrt_minmax_ and to a few ulp in scale_
 *                 (the two toolchains compile powf differently).
 *   MMB_DIV_IEEE  IEEE round-to-nearest division (formed exactly from a reciprocal and one correction step):
 *                 equals a CPU restatement bit for bit.  For the range-expansion format it also forms pow()
 *                 as 2^(y*log2 x) on the special-function unit when the exponent is at most 4 (within
 *                 ~1e-6 of the library powf: about 80 codes per million differ from the reference's).
 *   MMB_DIV_IEEE_STRICT  IEEE results through the compiler's division and the library powf everywhere:
 *                 slower, same bits as MMB_DIV_IEEE for the absmax format; exists to verify the fast exact
 *                 quotient against. */
#define MMB_DIV_IEEE 0
#define MMB_DIV_FULL 1
#define MMB_DIV_IEEE_STRICT 2

/* Newton-Schulz GEMM back ends */
#define MMB_NS_TCGEN05 0 /* tcgen05.mma + TMEM + TMA (the product).  Blocks with 64 < min(rows, cols) <= 128
                            and max(rows, cols) <= 384, and wide or square blocks with 128 < rows <= 256,
                            rows <= cols <= 256, run all five iterations in ONE launch, one CTA per block,
                            operands resident in shared and tensor memory; larger blocks run fifteen
                            batched GEMM launches                                                    */
#define MMB_NS_SIMT 1    /* plain CUDA-core tiles; slow, for cross-checking    */
#define MMB_NS_TCGEN05_MULTI 2 /* the fifteen-launch tensor-core path for every shape (for comparison) */

int mmb_version(void);
const char* mmb_last_error(void);
/* Launch options.  The four setters below act on the CALLING HOST THREAD only (like mmb_last_error and
 * mmb_set_device_grad_scale): they change how later calls of that thread size and schedule their kernels,
 * never what is computed.  Nothing else in the library is mutable state.
 *
 * Size every kernel's grid for at most n SMs (0 = all).  Leaving a few SMs
 * free lets communication kernels (NCCL) run beside the persistent GEMMs. */
int mmb_set_sm_limit(int n);
/* Cap the grids of the bandwidth-bound kernels (momentum, update, AdamW) at n CTAs per SM (0 = default: up to
 * 32 CTAs of 256 threads; values outside 0..32 are refused with MMB_ERR_INVALID).  With n > 0 the CTAs have
 * 128 threads and ask for the largest shared-memory carve-out, the shape that fits on an SM beside a
 * persistent GEMM CTA (one warp of at most 64 registers per sub-partition, no shared memory); with n = 1,
 * work issued on a second stream runs beside Newton-Schulz without taking SMs from it.  No counterpart in the
 * reference. */
int mmb_set_stream_ctas_per_sm(int n);
/* Tile schedule of the Newton-Schulz GEMMs (no counterpart in the reference).  0 (default): every CTA pair
 * takes tiles round-robin, fixed at launch.  1: pairs draw tile numbers from a counter in the workspace, so
 * a pair whose SMs are shared with another kernel (a collective running beside the step) takes fewer tiles
 * instead of delaying the launch.  Results do not depend on the schedule. */
int mmb_set_gemm_schedule(int dynamic);
/* How the Newton-Schulz GEMMs follow one another on their stream (no counterpart in the reference).
 * 1 (default): each GEMM is launched with programmatic stream serialisation; its CTAs may become resident
 * and set up their barriers and tensor memory while the previous kernel of the stream is finishing, and
 * wait (griddepcontrol.wait) for that kernel to complete before they touch global memory.  0: plain
 * launches.  Results do not depend on it. */
int mmb_set_gemm_dependent_launch(int on);
/* Kernels launched by this library in this process so far. */
int64_t mmb_launch_count(void);

/* ------------------------------------------------------------------------
 * Heavy-ball momentum with optimizer-state codec, fused:
 *   dequantise -> m = beta*m (rounded) -> m = m + round_gradtype(grad_scale*g) (rounded)
 *   -> requantise; also writes bf16(m) for Newton-Schulz and the per-block
 *   sum of squares of m.
 * Replaces: momentum update   pretrain/src/models/monarch/monarch_muon.py:146-148
 *                             membench/src/models/monarch/monarch_muon.py:150-151
 *           cat + bf16 cast   membench/.../monarch_muon.py:161-163
 *           FP8 state codec   pretrain/src/models/monarch/coat_state_muon.py:22-114
 *                             (expansion) and pretrain/third_party/coat/optimizer/
 *                             triton_kernels.py:34-36,51-63 (absmax)
 *           Frobenius norm    monarch_muon.py:38
 * One segment = one parameter tensor of nblocks blocks of block_elems
 * elements.  Groups of 128 restart at each segment; a tail group is masked.
 * ---------------------------------------------------------------------- */
typedef struct mmb_momentum_seg {
  const void* grad;     /* device, grad_dtype, [numel]                        */
  void* state;          /* device: E4M3 codes (uint8) or the bf16/fp32 buffer */
  float* scale;         /* device, [ceil(numel/128)]       (FP8 formats)      */
  float* expand;        /* device, [ceil(numel/128)]       (FP8_EXPAND only)  */
  float* sqrt_minmax;   /* device, [ceil(numel/128)]       (FP8_EXPAND only)  */
  void* m_bf16;         /* device, bf16 [numel], may be NULL                  */
  int64_t numel;        /* nblocks * block_elems                              */
  int64_t block_elems;  /* rows*cols of one block                             */
  int64_t first_block;  /* index of this segment's first block in block_sumsq */
} mmb_momentum_seg;

/* Number of floats of scratch (per-chunk partial sums) the call below needs. */
int64_t mmb_momentum_scratch_floats(const mmb_momentum_seg* segs, int nseg);

int mmb_momentum_step(const mmb_momentum_seg* segs, int nseg, int grad_dtype, int state_format,
                      int div_mode, float beta, float grad_scale, int expand_min,
                      float* block_sumsq_dev, /* [total blocks] or NULL           */
                      float* scratch_dev, int64_t scratch_floats, void* stream);

/* Same step for callers that cannot allocate device memory.  (No counterpart
 * in the reference; added for this library's users.)  Some hosts of this code
 * may not call cudaMalloc: a plugin running inside someone else's memory pool
 * or under a fixed device-memory budget, code on a latency-critical path where
 * an allocation could stall or fail, a process that has handed all free memory
 * to another allocator.  They still own gradients, state and outputs, but have
 * nowhere to put the kernel's scratch (one partial sum of squares per 4096
 * elements).  This entry point keeps that scratch in a fixed array compiled
 * into the library (4 MiB of device memory on every GPU that loads it, held
 * until the process exits) and calls no cudaMalloc, cudaFree or other
 * allocating routine.
 *   - Limit: mmb_momentum_static_max_floats() partial sums (2^20), i.e. tables
 *     for which mmb_momentum_scratch_floats() is larger are refused with
 *     MMB_ERR_INVALID and a message; about 4.29e9 state elements fit.
 *   - The first call on each device looks up the array's device address, with
 *     that device current; make that first call outside any stream capture.
 *     The address is remembered per device ordinal for the life of the process:
 *     after cudaDeviceReset() on that device the entry point must not be used
 *     again in the same process.
 *   - All calls on a device share the array.  It keeps whatever the last call
 *     left; nothing in it has to start at zero because every partial a call
 *     reads is written by that same call first.  Two calls whose kernels can
 *     overlap on the GPU (different streams) race on it - serialise them.
 * Arguments and results are exactly those of mmb_momentum_step. */
int64_t mmb_momentum_static_max_floats(void);
int mmb_momentum_step_static(const mmb_momentum_seg* segs, int nseg, int grad_dtype, int state_format,
                             int div_mode, float beta, float grad_scale, int expand_min,
                             float* block_sumsq_dev, void* stream);

/* Stand-alone codecs on one flat fp32 tensor (first-step quantise, state_dict
 * export, tests).  Replace coat_state_muon.py:94-114 (dequantize, quantize_). */
int mmb_fp8_quantize(const float* value_dev, uint8_t* codes_dev, float* scale_dev, float* expand_dev,
                     float* sqrt_minmax_dev, int64_t numel, int state_format, int is_signed,
                     int div_mode, int expand_min, void* stream);
int mmb_fp8_dequantize(const uint8_t* codes_dev, const float* scale_dev, const float* expand_dev,
                       const float* sqrt_minmax_dev, float* out_dev, int64_t numel, int state_format,
                       int is_signed, void* stream);

/* ------------------------------------------------------------------------
 * Batched quintic Newton-Schulz on `batch` bf16 blocks of rows x cols.
 * Replaces _newton_schulz_batched, monarch_muon.py:36-50 (bf16 twin:
 * membench/.../monarch_muon.py:36-50 with the cast at :161-166):
 *   X = B / (||B||_F + 1e-7); 5 x { A = X X^T; X = (aI + bA + cA^2) X }
 * computed on the stored orientation (tall blocks are never transposed in
 * memory), the polynomial in completed-square form c(A + b/2c I)^2 + (a -
 * b^2/4c) I so that each GEMM epilogue only scales and adds a diagonal.  The
 * norm prescale is applied inside the first iteration's epilogues.
 *   x_dev            bf16 [batch, rows, cols], input (momentum); also used as
 *                    scratch unless `out_dev` differs - see below
 *   out_dev          bf16 [batch, rows, cols]; may equal x_dev
 *   block_sumsq_dev  fp32 [batch] sum of squares per block, or NULL to have
 *                    the call compute it from x_dev
 *   workspace_dev    mmb_ns_workspace_bytes() bytes, 1024-byte aligned
 *   status_dev       int32 word from mmb_device_status_create(), or NULL
 * ---------------------------------------------------------------------- */
int64_t mmb_ns_workspace_bytes(int batch, int rows, int cols);
int mmb_newton_schulz(const void* x_dev, void* out_dev, const float* block_sumsq_dev, int batch,
                      int rows, int cols, void* workspace_dev, int64_t workspace_bytes, int backend,
                      int32_t* status_dev, void* stream);

/* Newton-Schulz and the Muon weight update in one call:
 *   W[b] <- W[b] + alpha * NS(X)[b],   alpha = -lr * sqrt(rows / cols)
 * Replaces _newton_schulz_batched followed by `param.data.add_(ortho, alpha=)`,
 * monarch_muon.py:36-50 and :160-165 (membench twin :167-170).  With the
 * tensor-core back end the update is the epilogue of the last GEMM: the
 * orthogonalised block never reaches memory; each result tile is rounded to bf16
 * (the value mmb_newton_schulz would store) and added to the weights with one
 * fused multiply-add and one rounding to the weights' type, exactly what the
 * stored result followed by mmb_muon_update gives.
 *   x_dev            bf16 [batch, rows, cols], only read
 *   weight_ptrs_dev  DEVICE array of `batch` pointers, entry b = block b's
 *                    rows x cols weights (row-major, 16-byte aligned)
 *   weight_dtype     MMB_BF16 or MMB_F32
 * Other arguments as for mmb_newton_schulz. */
int mmb_newton_schulz_update(const void* x_dev, const float* block_sumsq_dev, int batch, int rows, int cols,
                             void* const* weight_ptrs_dev, int weight_dtype, float alpha, void* workspace_dev,
                             int64_t workspace_bytes, int backend, int32_t* status_dev, void* stream);

/* One batched GEMM of the family Newton-Schulz is built from (exposed for
 * tests and profiling):
 *   D[b] = sigma_b * alpha * opA[b] . opB[b]^T + diag * I
 * opA is M x K, opB is N x K, D is bf16 [batch][M][N].  Operand modes:
 *   MMB_GEMM_K    stored [batch][rows][K] (K contiguous)
 *   MMB_GEMM_MN   stored [batch][K][rows] (rows contiguous)
 *   MMB_GEMM_SYM  symmetric rows x rows matrix of which only the 256 x 256
 *                 blocks on or above the block diagonal are read
 * sym_out != 0: D is symmetric and only those blocks of it are written.
 * sigma_b = inv_norm[b]^sigma_pow (sigma_pow 0: 1). */
/* Diagnostic: CTAs (pair = 0) or two-CTA clusters (pair = 1) of the 256-wide
 * GEMM kernel that fit on the current device at once. */
int mmb_gemm_occupancy(int pair, int* out);
#define MMB_GEMM_K 0
#define MMB_GEMM_MN 1
#define MMB_GEMM_SYM 2
int mmb_gemm_bf16(const void* a_dev, const void* b_dev, void* d_dev, int batch, int M, int N, int K,
                  int a_mode, int b_mode, int sym_out, float alpha, float diag,
                  const float* inv_norm_dev, int sigma_pow, int backend, int32_t* status_dev,
                  void* stream);

/* ------------------------------------------------------------------------
 * Muon weight update, W <- W + alpha * O with alpha = -lr*sqrt(rows/cols).
 * Replaces monarch_muon.py:160-165 (membench :167-170).
 * ---------------------------------------------------------------------- */
typedef struct mmb_update_seg {
  void* weight;       /* device, weight_dtype, [numel]      */
  const void* ortho;  /* device, bf16, [numel]              */
  int64_t numel;
} mmb_update_seg;

int mmb_muon_update(const mmb_update_seg* segs, int nseg, int weight_dtype, float alpha, void* stream);

/* ------------------------------------------------------------------------
 * Decoupled AdamW over a list of tensors, one launch per <=128 tensors.
 * Replaces _adamw_step, monarch_muon.py:171-201 (membench :176-208): weight
 * decay multiplies the parameter first; eps is added after sqrt(v)/sqrt(bc2);
 * every intermediate is rounded to the tensor dtype like the reference's
 * separate torch ops.  `step` is the already-incremented count.  The
 * hyper-parameters of this and the two other AdamW entries are doubles, the
 * reference's Python floats: 1 - lr*wd, 1 - beta, sqrt(1 - beta2^step) and
 * lr / (1 - beta1^step) are formed in double as the reference forms them and
 * narrowed once to fp32, as torch narrows a Python scalar (1 - 0.9 taken from
 * a float 0.9 would be three ulps away from torch's alpha).
 * ---------------------------------------------------------------------- */
typedef struct mmb_adamw_seg {
  void* param;        /* device, dtype */
  const void* grad;   /* device, dtype */
  void* exp_avg;      /* device, dtype */
  void* exp_avg_sq;   /* device, dtype */
  int64_t numel;
  int32_t step;       /* per tensor (the pretrain twin counts per parameter) */
  int32_t pad_;
} mmb_adamw_seg;

int mmb_adamw_step(const mmb_adamw_seg* segs, int nseg, int dtype, double lr, double beta1, double beta2,
                   double weight_decay, double eps, void* stream);

/* ------------------------------------------------------------------------
 * AdamW with both moments stored as E4M3 codes + per-128-group side arrays,
 * decoded, stepped and re-encoded in one pass.  Replaces the AdamW part of
 * CoatStateMonarchMuon.step, pretrain/src/models/monarch/coat_state_muon.py:
 * 126-139 (dequantize every state -> _adamw_step, monarch_muon.py:171-201,
 * with fp32 moments -> quantize_): exp_avg is a signed state, exp_avg_sq an
 * unsigned one (:19).  state_format is MMB_STATE_FP8_EXPAND (the reference's
 * codec; expand_* and sqrt_minmax_* required) or MMB_STATE_FP8_ABSMAX (they
 * may be NULL).  Fresh states are all-zero codes with side arrays set to 1.
 * ---------------------------------------------------------------------- */
typedef struct mmb_adamw_fp8_seg {
  void* param;                   /* device, dtype                     */
  const void* grad;              /* device, dtype                     */
  void* exp_avg;                 /* device, E4M3 codes [numel]        */
  float* scale_exp_avg;          /* device, fp32 [ceil(numel/128)]    */
  float* expand_exp_avg;
  float* sqrt_minmax_exp_avg;
  void* exp_avg_sq;              /* device, E4M3 codes [numel]        */
  float* scale_exp_avg_sq;
  float* expand_exp_avg_sq;
  float* sqrt_minmax_exp_avg_sq;
  int64_t numel;
  int32_t step;                  /* already-incremented count         */
  int32_t pad_;
} mmb_adamw_fp8_seg;

int mmb_adamw_fp8_step(const mmb_adamw_fp8_seg* segs, int nseg, int dtype, int state_format, int div_mode, double lr,
                       double beta1, double beta2, double weight_decay, double eps, int expand_min, void* stream);

/* ------------------------------------------------------------------------
 * Steps on fp32 master weights with a bf16 copy for the model, as the
 * reference's fine-tuning optimizer keeps them (finetune/sft_optimizer.py:33-59:
 * state["master"] is updated, then `p.copy_(master)`).  Update and down-cast
 * are one pass.  `shadow` may be NULL (no copy written).
 *   mmb_muon_update_master: master <- master + alpha*O       (:48-49)
 *   mmb_adamw_master_step : torch.optim AdamW on the master  (:51-55), in the
 *     arithmetic of torch's fused CUDA kernel, which is what that call runs on
 *     a GPU (fp32 hyper-parameters, 1 - beta from the float beta, bias
 *     corrections by the float power function): bit-exact with the reference
 *     class on the GPU; moments are fp32, the gradient is read in its own dtype
 *     (`p.grad.float()`, :44), `step` is the already-incremented count.
 * ---------------------------------------------------------------------- */
typedef struct mmb_master_update_seg {
  void* master;       /* device, fp32, [numel]              */
  void* shadow;       /* device, bf16, [numel] or NULL      */
  const void* ortho;  /* device, bf16, [numel]              */
  int64_t numel;
} mmb_master_update_seg;

int mmb_muon_update_master(const mmb_master_update_seg* segs, int nseg, float alpha, void* stream);

typedef struct mmb_master_adamw_seg {
  void* master;       /* device, fp32                       */
  void* shadow;       /* device, bf16 or NULL               */
  const void* grad;   /* device, grad_dtype                 */
  void* exp_avg;      /* device, fp32                       */
  void* exp_avg_sq;   /* device, fp32                       */
  int64_t numel;
  int32_t step;
  int32_t pad_;
} mmb_master_adamw_seg;

int mmb_adamw_master_step(const mmb_master_adamw_seg* segs, int nseg, int grad_dtype, double lr, double beta1,
                          double beta2, double weight_decay, double eps, void* stream);

/* ------------------------------------------------------------------------
 * Global gradient norm and clip coefficient, computed on the device with no
 * host round trip.  Replaces torch.nn.utils.clip_grad_norm_ in the training
 * loop (pretrain/src/optim/base.py:121-122: the norm's .item() is a host sync,
 * and the in-place scaling of every gradient is two more passes over them).
 *   out_dev[0] = ||all gradients||_2, out_dev[1] = min(1, max_norm/(norm+1e-6)).
 * mmb_set_device_grad_scale(&out_dev[1]) then makes the following
 * mmb_momentum_step / mmb_adamw_step calls of this thread multiply every
 * gradient by that device scalar as they read it (NULL switches it off), so the
 * gradients themselves are never rewritten.
 * ---------------------------------------------------------------------- */
typedef struct mmb_grad_seg {
  const void* grad; /* device */
  int64_t numel;
  int32_t dtype;    /* MMB_BF16 or MMB_F32 */
  int32_t pad_;
} mmb_grad_seg;

int64_t mmb_grad_norm_scratch_floats(void);
int mmb_grad_norm_clip(const mmb_grad_seg* segs, int nseg, float max_norm, float* out_dev,
                       float* scratch_dev, int64_t scratch_floats, void* stream);
int mmb_set_device_grad_scale(const float* scale_dev);

/* ------------------------------------------------------------------------
 * Reduce-scatter / all-gather pieces of the data-parallel (owner-computes) step
 * through NVSwitch multicast.  No counterpart in the reference, which all-reduces
 * gradients with DDP and steps every parameter on every rank
 * (pretrain/src/distributed/ddp.py:42-52).  Both calls take one address inside a
 * MULTICAST mapping of a buffer that every GPU of the group holds at the same
 * offset (torch.distributed's symmetric memory provides it) and one ordinary
 * device address, `nbytes` a multiple of 16, all 16-byte aligned:
 *   mmb_multimem_reduce_bf16  dst[i] = sum over the group's copies of src[i], bf16
 *                             elements added with fp32 accumulation inside the
 *                             switch (multimem.ld_reduce) - called on the range a
 *                             rank owns, this is its share of a reduce-scatter;
 *   mmb_multimem_broadcast    every copy of dst[i] = src[i] (multimem.st) - called
 *                             on the range a rank owns, its share of an all-gather.
 * `ctas` CTAs of 128 threads are launched.  They are small on purpose (no shared
 * memory, at most 64 registers): one such CTA fits on an SM beside a Newton-Schulz
 * GEMM CTA, so the transfer shares SMs with the GEMMs instead of taking SMs from
 * them; use at most one CTA per SM.  The kernels wait on nothing and hold no
 * flags: the caller orders them against the other ranks (all copies written before
 * the first reduce; a group-wide collective after the last broadcast before any
 * copy is read).  On a GPU or buffer without multicast support the calls must not
 * be used.
 * ---------------------------------------------------------------------- */
int mmb_multimem_reduce_bf16(const void* multicast_src, void* dst_dev, int64_t nbytes, int ctas, void* stream);
int mmb_multimem_broadcast(const void* src_dev, void* multicast_dst, int64_t nbytes, int ctas, void* stream);
/* The same two pieces over plain peer addresses (no multicast object needed; no counterpart in the
 * reference).  `copies` is a HOST array of device addresses, each 16-byte aligned, that this GPU can
 * reach (its own memory or a peer mapping, e.g. symmetric memory's per-rank buffer pointers):
 *   mmb_peer_reduce_bf16  dst[i] = bf16(copies[0][i] + copies[1][i] + ... ), bf16 elements, fp32
 *                         accumulation in the order given, one rounding; `world` in 1..16;
 *   mmb_peer_broadcast    copies[r][i] = src[i] for r < count (leave this GPU's own copy out when src
 *                         already is it); `count` in 0..16.
 * Same CTA shape, same ordering contract as the multicast calls. */
int mmb_peer_reduce_bf16(const void* const* copies, int world, void* dst_dev, int64_t nbytes, int ctas, void* stream);
int mmb_peer_broadcast(const void* src_dev, void* const* copies, int count, int64_t nbytes, int ctas, void* stream);

/* ------------------------------------------------------------------------
 * Device status word.  Kernels never trap: a bounded wait that expires or a
 * failed self-check stores a non-zero code here and the kernel returns.
 * mmb_device_status_read synchronises `stream` and returns the word.
 * ---------------------------------------------------------------------- */
/* Status codes a kernel may store (0 = nothing to report). */
#define MMB_STATUS_WAIT_PRODUCER_EMPTY 0x101 /* a TMA producer waited too long for a free stage            */
#define MMB_STATUS_WAIT_MMA_FULL 0x102       /* the MMA issuer waited too long for operands                 */
#define MMB_STATUS_WAIT_MMA_TMEM_EMPTY 0x103 /* the MMA issuer waited too long for a drained accumulator     */
#define MMB_STATUS_WAIT_EPI_TMEM_FULL 0x104  /* an epilogue warp waited too long for an accumulator          */
#define MMB_STATUS_WAIT_SCHED_FULL 0x105     /* a role waited too long for its next tile number              */
#define MMB_STATUS_WAIT_SCHED_EMPTY 0x106    /* the tile scheduler waited too long for a slot                */
#define MMB_STATUS_WAIT_PROBE 0x1F0          /* mmb_wait_probe: the unanswered wait expired, as it must      */
int mmb_device_status_create(int32_t** status_dev_out);
int mmb_device_status_destroy(int32_t* status_dev);
int mmb_device_status_read(int32_t* status_dev, int32_t* host_out, int reset, void* stream);
/* Self-test of the bounded wait (no counterpart in the reference): launches one warp that waits, with the
 * same wait routine the GEMM roles use and a limit of `limit_cycles` SM cycles (1 .. 2e9), on a barrier that
 * nothing ever arrives at.  The wait expires, the kernel stores MMB_STATUS_WAIT_PROBE in the status word
 * and returns; the device stays usable.  Nothing faults, traps or hangs. */
int mmb_wait_probe(int64_t limit_cycles, int32_t* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MONARCH_MUON_B200_H */
