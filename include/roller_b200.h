/*
 * roller_b200 -- C ABI of the B200 (sm_100a) backend for the Roller rTile search -> fp32 GEMM path.
 *
 * The reference project compiles one `gemm_kernel(float* A, float* B, float* C)` per search hint
 * through an MLIR/IREE pipeline and launches it through CuPy (src/roller.py:345-387 Compiler,
 * src/roller.py:499-511 prepare_kernel, src/roller.py:525-607 run_eval / run_baseline). This
 * library replaces that compile-and-launch layer: kernels are ahead-of-time compiled for
 * sm_100a, one per buildable rTile, and a "plan" binds an rTile to a problem shape.
 *
 * Conventions
 *   - every function returns 0 (ROLLER_OK) or a negative roller_status; nothing throws, aborts
 *     or exits across this boundary;
 *   - A is M x K, B is K x N, C is M x N, all row-major in device memory owned by the caller
 *     (fp32, or 16-bit floats in the 16-bit modes); lda/ldb/ldc are row strides in elements;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream); *_run only
 *     enqueues work;
 *   - a plan is bound to the device that was current at create time and is not thread-safe;
 *     launches of one plan must also be ordered on the device (same stream, or streams ordered
 *     by events): a plan owns one staging area, one stream-K scratch area and one status word.
 *     Use one plan per stream to overlap GEMMs;
 *   - a launch is a persistent grid (at most one CTA per SM) whose CTAs may wait for one
 *     another when leftover tiles are split along K, so all of them must get an SM eventually:
 *     a kernel on another stream that occupies SMs must not itself wait for this launch. Every
 *     such wait is bounded (~2 s) and ends in ROLLER_ERR_TIMEOUT rather than a hang.
 */
#ifndef ROLLER_B200_H_
#define ROLLER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum roller_status {
  ROLLER_OK = 0,
  ROLLER_ERR_INVALID = -1,     /* bad argument (null pointer, non-positive size, bad stride) */
  ROLLER_ERR_UNSUPPORTED = -2, /* no compiled kernel for the requested rTile / mode */
  ROLLER_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed; see roller_b200_last_cuda_error */
  ROLLER_ERR_DEVICE = -4,      /* the current device is not an sm_100 part, or not the plan's device */
  ROLLER_ERR_TIMEOUT = -5,     /* a bounded device-side wait ran out; see roller_b200_last_status */
  ROLLER_ERR_NOMEM = -6,       /* workspace allocation failed */
  ROLLER_ERR_TOO_LARGE = -7    /* problem exceeds a fixed capacity of the entry point */
} roller_status;

/* Arithmetic modes of the tensor-core GEMM. */
#define ROLLER_MODE_1XTF32 1 /* one TF32 product per fp32 product (10-bit mantissa inputs) */
#define ROLLER_MODE_3XTF32 3 /* big/small split, three TF32 products: fp32-level accuracy */
/* 16-bit operands: A and B hold bf16 / fp16 elements (leading dimensions in elements), products
 * are exact, accumulation and C are fp32. The reference's MatmulConfig carries the element width
 * (el_bits, src/analyze.py:31,39-41); its kernel generator only emits f32 (src/roller.py:47-68). */
#define ROLLER_MODE_BF16 16
#define ROLLER_MODE_F16 17

/* Flags for roller_b200_gemm_create. */
#define ROLLER_FLAG_ACCUMULATE 1 /* C += A@B, the semantics of the reference's gemm_kernel, which
                                    accumulates into a host-zeroed C (src/roller.py:62,534) */
#define ROLLER_FLAG_B_TRANSPOSED 2 /* B is passed as Bt[N,K] row-major (ldb >= K); the reference's
                                      cost model already treats B that way (src/analyze.py:33-34)
                                      and its tutorial kernels pre-transpose B
                                      (src/cuda_matmul_opt.py:280-281,376-392) */

#define ROLLER_FLAG_C_16BIT 4 /* 16-bit modes only: C (and ldc) are in the operand type as well, as
                                 the reference's MatmulConfig implies for its output tensor
                                 (one el_bits for A, B and C, src/analyze.py:31-49); sums are
                                 kept in fp32 and rounded to nearest even once, on the store */

/* Options of roller_b200_gemm_set_option. */
#define ROLLER_OPT_WAIT_LIMIT_CYCLES 1 /* clock cycles any device-side wait of the plan's launches
                                          may last before the kernel gives up (0 = the default,
                                          about two seconds) */
#define ROLLER_OPT_OVERLAP_LAUNCH 2    /* 1 (default): launches carry the programmatic-stream-
                                          serialization attribute, so a launch is scheduled while
                                          the previous kernel of its stream winds down and sets up
                                          its CTAs early; it still waits for that kernel's
                                          completion before touching global memory. 0: plain
                                          stream order */
#define ROLLER_OPT_TMA_STORE 3         /* C leaves each CTA through shared memory and TMA stores
                                          instead of the accumulate warps' own stores, so a slow
                                          destination (C in another GPU's memory, mapped into
                                          this process) does not hold the warps up. The library
                                          uses this path by itself where it can: fp32 C with
                                          16-byte aligned base and row stride, no
                                          ROLLER_FLAG_ACCUMULATE, an rTile whose kernel has the
                                          staging area. 1 insists on it (ROLLER_ERR_UNSUPPORTED /
                                          _INVALID where it cannot work); 0 turns it off */
#define ROLLER_OPT_PROGRESSIVE_ROUNDS 4 /* n > 0: every tile is cut along K and the tiles are
                                          worked through in n groups by the whole grid, so that
                                          finished tiles leave the kernel at a steady rate from
                                          early on rather than together at the end (at most 16,
                                          and at most one per tile). -1 = the library picks n;
                                          0 = off. With equal rounds of fewer tiles than CTAs
                                          (or CTA pairs) the grid shrinks by up to a sixth to a
                                          count that the tiles of a round divide */
#define ROLLER_OPT_ROUND_RATIO 7        /* size of each round of the progressive schedule relative
                                          to the one before it, in percent (25 .. 400; default
                                          100 = equal rounds). When C leaves over a link while
                                          the computation goes on, the time to the last byte is
                                          shortest with a ratio of about t_link / t_compute:
                                          shrinking rounds when the computation is the longer of
                                          the two (little is left to send after the last round),
                                          growing ones when the link is (it starts early) */
#define ROLLER_OPT_EARLY_EXIT 8         /* 1: with TMA stores, a CTA leaves as soon as the TMA unit
                                          has read its last tile from shared memory instead of
                                          waiting for the stores to be performed; C is complete
                                          when the kernel is (stream order), and a kernel of
                                          another stream can take the SM meanwhile. Ignored by a
                                          launch that raises an arrival flag itself. Default 0 */
#define ROLLER_OPT_COOPERATIVE_FIXUP 6  /* 1 (default): in the progressive schedule with TMA stores a
                                          tile shared by several workers is completed by all of
                                          them together, each adding a slice of everybody's
                                          partial sums; 0: by the worker holding the end of its
                                          reduction alone, as the plain stream-K schedule does */
#define ROLLER_OPT_TEST_DROP_PUBLISH 5 /* test aid, 1: workers that hand a partial tile to another
                                          worker write it but never raise its flag, so the bounded
                                          wait of the receiving worker runs out and the launch ends
                                          with ROLLER_ERR_TIMEOUT. Nothing faults or hangs */

/* Most flags one roller_b200_flag_signal_async call can raise. */
#define ROLLER_MAX_FLAG_TARGETS 32

/* Device facts feeding the B200 device model of the search (reference: the constants hard-coded
 * in arch.CUDA, src/arch.py:47-61). */
typedef struct roller_dev_info {
  int cc_major, cc_minor;
  int sm_count;
  int smem_per_block_optin; /* bytes a block may opt in to */
  int smem_per_sm;          /* bytes */
  int regs_per_sm;
  int l2_bytes;
  int sm_clock_khz;
  int mem_clock_khz;
  int mem_bus_bits;
  int tmem_columns; /* 512 columns x 128 lanes x 32 bit per SM on sm_100 */
  size_t total_mem;
  char name[128];
} roller_dev_info;

/* One buildable rTile = one compiled kernel (reference: a TileDict hint, src/analyze.py:84-105,
 * handed to Compiler, src/roller.py:345-356). */
typedef struct roller_ktile {
  int block_m;   /* output tile rows (128 per CTA, 256 for a CTA pair) */
  int block_n;   /* output tile columns */
  int rstep;     /* reduce step per pipeline stage, in fp32 elements (one 128-byte row) */
  int cta_group; /* 1, or 2 = two SMs cooperate on one tile (tcgen05 cta_group::2) */
  int stages_1x; /* pipeline depth in 1xTF32 mode */
  int stages_3x; /* pipeline depth in 3xTF32 mode */
  int smem_1x;   /* dynamic shared memory per CTA, bytes */
  int smem_3x;
  int tmem_cols; /* TMEM columns allocated (double-buffered accumulator) */
  int threads_1x;
  int threads_3x;
  int layout;    /* 0 = general tile; 2 = "skinny": for a C with few rows the tensor core works on
                    C^T, block_m (32 or 64) rows of C by block_n = 128 columns per tile;
                    3 = "skinny" on the CUDA cores: plain fp32 FMAs, 16 rows of C by 256 columns
                    per CTA, split along K. It exists for ROLLER_MODE_3XTF32 only (stages_1x =
                    0): its results are fp32-exact products, which is what that mode promises */
  int rstep_16;  /* reduce step of the tile's kernel for 16-bit operands, in elements (64);
                    0 = the tile has no such kernel */
  int stages_16; /* its pipeline depth and dynamic shared memory */
  int smem_16;
} roller_ktile;

typedef struct roller_plan roller_plan;

/* Replaces the constants of arch.CUDA (src/arch.py:47-61) with a query of device `dev`. */
int roller_b200_device_info(int dev, roller_dev_info* out);

/* Enumerate the compiled rTiles, so the search only emits hints that have a kernel (the
 * reference can compile any hint at run time, src/roller.py:358-387). */
int roller_b200_kernel_count(void);
int roller_b200_kernel_desc(int idx, roller_ktile* out);

/* Replaces Compiler(config, hint, ...).compile() (src/roller.py:345-387): bind an rTile to a
 * problem. May allocate device workspace (only when the rows of A or B are not multiples of 16
 * bytes long, in which case operands are staged through a padded copy). `mode` also fixes the
 * operand element type: fp32 for the TF32 modes, bf16 / fp16 for ROLLER_MODE_BF16 / _F16. */
int roller_b200_gemm_create(const roller_ktile* tile, int M, int N, int K, int lda, int ldb,
                            int ldc, int mode, int flags, roller_plan** out);

/* Replaces cuda_func(grid, block, (A, B, C), shared_mem=...) (src/roller.py:545-550): enqueue one
 * GEMM on `stream`. No allocation, no synchronisation. A and B point to elements of the type
 * the plan's mode names; C is fp32 unless the plan was made with ROLLER_FLAG_C_16BIT. Because
 * it only enqueues, the call may be made on a capturing stream; replays of the captured graph
 * run the same launch on the same pointers (tested with the stream-K schedule active). */
int roller_b200_gemm_run(roller_plan* plan, const void* A, const void* B, void* C, void* stream);

/* Replaces the timed loop of run_eval (src/roller.py:564-584): `warmup` untimed launches, then
 * `iters` launches between two CUDA events on `stream`; *ms_per_iter is the mean. Blocks. */
int roller_b200_gemm_time(roller_plan* plan, const void* A, const void* B, void* C, void* stream,
                          int warmup, int iters, float* ms_per_iter);

/* Host-buffer form of the whole run_eval data path -- allocate/upload operands, launch, read C
 * back (src/roller.py:532-550) -- used for end-to-end timing: copies A and B from host memory into
 * plan-owned device buffers, runs the GEMM and copies C back, all on `stream`; blocks until C
 * has arrived. The device buffers are allocated on the first call and kept. */
int roller_b200_gemm_host(roller_plan* plan, const void* hA, const void* hB, void* hC,
                          void* stream);

/* Same data path as roller_b200_gemm_host (src/roller.py:532-550) without the final wait: the
 * copies and the launch are only enqueued on `stream`, so GEMMs on different streams overlap
 * their uploads, kernels and readbacks. Host buffers should be pinned; hC is valid once `stream`
 * has been synchronised. */
int roller_b200_gemm_host_async(roller_plan* plan, const void* hA, const void* hB, void* hC,
                                void* stream);

/* Copies a rows x cols block of fp32 between two device matrices (leading dimensions in
 * elements) with the driver's copy engines, enqueued on `stream`; either side may be another
 * GPU's memory mapped into this process. The multi-GPU driver uses it to push a finished band of
 * C into the destination rank's matrix while the next band is still being computed. There is
 * no counterpart in the reference, which runs on one device (.env:5-6). */
int roller_b200_copy_block_async(float* dst, long long dst_ld, const float* src, long long src_ld,
                                 long long rows, long long cols, void* stream);

/* Launch geometry the plan chose (the reference derives grid/block from the hint,
 * src/roller.py:536-543). Any out pointer may be NULL. */
int roller_b200_gemm_launch_info(const roller_plan* plan, int* grid, int* block, int* smem_bytes,
                                 int* tiles_m, int* tiles_n, int* max_clusters);

/* How the plan deals its work out, which the reference fixes at one block per tile
 * (src/roller.py:536): tiles cut along K (0 = none), the rounds they are worked through in
 * (1 unless the progressive schedule is on), and the k-blocks per schedule unit and per
 * accumulation chunk. Any out pointer may be NULL. */
int roller_b200_gemm_schedule_info(const roller_plan* plan, int* sk_tiles, int* rounds,
                                   int* unit_kb, int* chunk_kb);

/* The rounds of the progressive schedule: writes the first tile of each round followed by the
 * number of tiles cut along K into tile_begin[0 .. rounds] (`capacity` >= rounds + 1 entries,
 * else ROLLER_ERR_INVALID). The reference has one block per tile and no rounds
 * (src/roller.py:536). */
int roller_b200_gemm_round_tiles(const roller_plan* plan, int* tile_begin, int capacity);

/* Accumulation chunk of the 3xTF32 mode: the TMEM accumulator is drained into fp32 registers
 * every `k_elems` elements of the reduction (rounded up to whole 32-element steps; 0 = never,
 * one chunk spans K). Shorter chunks cost more drains and give a smaller rounding error. The
 * reference's kernels accumulate in fp32 registers throughout (src/roller.py:280-282). */
int roller_b200_gemm_set_chunk(roller_plan* plan, int k_elems);

/* Overrides the number of persistent CTAs (a multiple of cta_group, at most the SM count and
 * at most one per tile). The reference derives its grid from the hint (src/roller.py:536). */
int roller_b200_gemm_set_grid(roller_plan* plan, int ctas);

/* Stream-K scheduling of the leftover tiles (those that do not fill a last wave of the persistent
 * grid; they are dealt out along K in pieces of one accumulation chunk in 3xTF32, of 8 k-blocks
 * in the other modes): -1 = use it when it shortens the schedule by 3 % or more (default), 0 = never (every
 * tile is reduced by one worker; results are then bit-identical for every rTile and every
 * sharding), 1 = whenever there are leftover tiles. May allocate the scratch area for the
 * partial tiles. The reference's grid is always one block per tile (src/roller.py:536). */
int roller_b200_gemm_set_stream_k(roller_plan* plan, int mode);

/* Sets one option of a plan (ROLLER_OPT_*); affects later launches. The reference has no
 * run-time options: its schedule is fixed when a hint is compiled (src/roller.py:93-342). */
int roller_b200_gemm_set_option(roller_plan* plan, int option, long long value);

/* Raises flags in other GPUs' memory: stores `value` (system-scope release) into each of the
 * `n` addresses in `targets` (host array of device pointers, each possibly another GPU's memory
 * mapped into this process), enqueued on `stream` behind the work whose completion it announces.
 * The multi-GPU driver uses it to tell the rank that collects C that this rank's stores have
 * landed, and to release the other ranks into the next step. There is no counterpart in the
 * reference, which runs on one device (.env:5-6). */
int roller_b200_flag_signal_async(uint32_t* const* targets, int n, uint32_t value, void* stream);

/* roller_b200_gemm_run with the hand-shake of a multi-GPU step carried out by the kernel itself,
 * for a C that is another GPU's memory: no store into C leaves before the word at `go_flag`
 * (this GPU's memory; the other GPU raises it when it is done with the previous contents of C)
 * has reached `go_value`, and once all stores of the launch have been performed `arrive_value`
 * is stored (system-scope release) into `arrive_flag` (normally the other GPU's memory). Either
 * pointer may be null. The wait for "go" sits in front of the first store, so the first tiles
 * are computed meanwhile; it is bounded like every device-side wait (ROLLER_OPT_WAIT_LIMIT_CYCLES):
 * when it runs out the launch is reported by roller_b200_last_status and raises no flag.
 * ROLLER_ERR_UNSUPPORTED unless the plan writes C through the TMA-store output path
 * (ROLLER_OPT_TMA_STORE); the caller then brackets roller_b200_gemm_run with
 * roller_b200_flag_wait_async / roller_b200_flag_signal_async. There is no counterpart in the
 * reference, which runs on one device (.env:5-6). */
int roller_b200_gemm_run_synced(roller_plan* plan, const void* A, const void* B, void* C,
                                const uint32_t* go_flag, uint32_t go_value, uint32_t* arrive_flag,
                                uint32_t arrive_value, void* stream);

/* Enqueues a one-block kernel that waits until each of the first `n` (<= 64) words of `flags`
 * selected by `mask` (bit i = word i) has reached `value` (flags count steps; the comparison
 * survives wrap-around). The wait is bounded: after `limit_cycles` clock cycles (0 = about two
 * seconds) the kernel stores a non-zero code into *dev_status (device memory, zeroed by the
 * caller) and returns, so a rank that never signals costs a time-out, not a hang. There
 * is no counterpart in the reference (single device, .env:5-6). */
int roller_b200_flag_wait_async(const uint32_t* flags, int n, unsigned long long mask,
                                uint32_t value, long long limit_cycles, uint32_t* dev_status,
                                void* stream);

/* One GEMM, enqueued on `stream`, that allocates nothing: no cudaMalloc, cudaFree or allocating
 * library call, on this or any later call. It has no counterpart in the reference (whose launch
 * path allocates freely through CuPy); it exists for callers that cannot allocate -- a process
 * whose own memory pool already holds all of the device's memory, or a latency-critical loop that
 * cannot afford the implicit device synchronisation of cudaMalloc/cudaFree.
 * It does what roller_b200_gemm_create + roller_b200_gemm_run do, including the padded staging
 * copies for operands whose row stride or base address is not a multiple of 16 bytes, but keeps
 * that scratch in a fixed 32 MiB array inside the library (resident on every GPU that loads the
 * library, until exit). Staging needs beyond 32 MiB return ROLLER_ERR_TOO_LARGE.
 * All calls share the array and it keeps the last call's contents: calls whose GPU work
 * overlaps race on it. The first call on a device resolves the array's device address; make
 * that call before starting any stream capture. Under CUDA's default lazy module loading the
 * array and each kernel image receive their device memory at first use, so a caller whose pool
 * will take all device memory should make one call per rTile and mode beforehand (or set
 * CUDA_MODULE_LOADING=EAGER). `dev_status` (optional, device memory) receives
 * the kernel's bounded-wait status word; NULL uses a word inside the library. C = A @ B. */
int roller_b200_gemm_static_scratch(const roller_ktile* tile, int mode, int M, int N, int K,
                                    int lda, int ldb, int ldc, const float* A, const float* B,
                                    float* C, uint32_t* dev_status, void* stream);

/* Stands in for the per-hint try/except of the sweep (src/benchmark.py:43-58): a kernel whose
 * pipeline stalls ends by itself and reports here instead of hanging.
 * Reads back the device status word of the plan (0 = all bounded waits completed); returns
 * ROLLER_ERR_TIMEOUT when it is non-zero. Synchronises the device. A non-zero word is cleared
 * by this call (with the plan's stream-K flags), so the plan can be launched again; until it has
 * been read, later launches of the plan give up at their first wait and leave C undefined, which
 * is why callers that time or compare kernels must read it after they have run them. */
int roller_b200_last_status(roller_plan* plan, uint32_t* device_status);

/* Releases what roller_b200_gemm_create allocated (the reference leaves its module to the
 * garbage collector, src/roller.py:504-505). */
int roller_b200_gemm_destroy(roller_plan* plan);

/* Text for a roller_status; the Python layer raises it as the exception message that the
 * sweep prints per failed hint (src/benchmark.py:55-58). */
const char* roller_b200_strerror(int status);
/* Text of the last CUDA error seen by this library on the calling thread (the reference
 * surfaces CuPy's exception text the same way, src/benchmark.py:55-58). */
const char* roller_b200_last_cuda_error(void);

#ifdef __cplusplus
}
#endif

#endif /* ROLLER_B200_H_ */
