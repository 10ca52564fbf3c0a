// Host-side table of the compiled GEMM kernels (one per rTile x mode) and their launcher.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace rb200 {

// Default limit of every device-side wait, in clock cycles: about two seconds at the B200's
// boost clock; no legitimate wait in these kernels lasts longer than a few milliseconds. The
// host may pass a shorter limit per launch.
constexpr long long kSpinLimitCycles = 4000000000LL;

// Kernel flag bits (GemmArgs::flags).
constexpr int kFlagAccumulate = 1;  // C += A@B instead of C = A@B
constexpr int kFlagVecStore = 2;    // C rows are 16-byte aligned: use 128-bit stores
constexpr int kFlagC16 = 4;         // 16-bit kernels only: C holds elements of the operand type
constexpr int kFlagTmaStore = 8;    // C leaves through shared memory and TMA stores (GemmArgs::tmC)
constexpr int kFlagCoopFixup = 32;  // shared tiles are completed by all their workers together (needs
                                    // kFlagTmaStore; four scratch slots and reader counts per CTA)
constexpr int kFlagSmemStore = 128; // fp32 C whose rows are not 16-byte aligned: tiles are turned
                                    // through the staging area so that a warp writes 32
                                    // consecutive floats of one row per store (needs the
                                    // staging area; not together with kFlagTmaStore)
constexpr int kFlagEarlyExit = 256; // with kFlagTmaStore: a CTA leaves once the TMA unit has read its
                                    // last tile from shared memory; the stores are complete
                                    // when the kernel is, so the next kernel of another stream
                                    // can take the SM while they are still on their way
constexpr int kFlagPeerSync = 64;   // the launch waits for and raises another GPU's flags itself
                                    // (GemmArgs::peer; needs kFlagTmaStore)
constexpr int kFlagDropPublish = 16;  // test aid: partial tiles are written but never flagged, so
                                      // the worker completing the tile sees its bounded wait run out

// Hand-shake of one launch with another GPU of the node, carried out by the kernel itself (with
// kFlagPeerSync, TMA-store output path only). `go_flag` (this GPU's memory) must have reached
// `go_value` before the first store into C leaves; once every store of the launch has been
// performed, `arrive_value` is stored -- release, system scope -- into `arrive_flag` (normally
// the other GPU's memory). Either pointer may be null. `arrive_count` is a word of this GPU
// that counts the warps done with their stores; the last one raises the flag and leaves zero.
struct PeerSync {
  const uint32_t* go_flag;
  uint32_t* arrive_flag;
  uint32_t* arrive_count;
  uint32_t go_value;
  uint32_t arrive_value;
};

// Rounds of the progressive schedule: round r owns the stream-K tiles
// [tile_begin[r], tile_begin[r + 1]); tile_begin[rounds] = sk_tiles. Unused with one round.
constexpr int kMaxRounds = 16;
struct RoundPlan {
  int tile_begin[kMaxRounds + 1];
};

struct GemmArgs {
  CUtensorMap tmA;
  CUtensorMap tmB;
  CUtensorMap tmC;      // C as a store destination (32 x 32 boxes); used with kFlagTmaStore only
  float* C;
  int M, N, K;
  long long ldc;
  int tiles_m, tiles_n;
  int chunk_kb;  // unit of the stream-K schedule, in k-blocks
  int acc_kb;    // k-blocks accumulated in TMEM before a drain into registers
  int flags;
  uint32_t* status;
  long long spin_limit; // clock cycles a device-side wait may last
  bool serialize_programmatically;  // launch may overlap the tail of the stream's previous kernel
  int sk_tiles;         // tiles dealt out in k-chunks (stream-K); 0 = whole tiles only
  int sk_rounds;        // groups the stream-K tiles are worked through one after the other (>= 1)
  float* sk_ws;         // four 128 x block_n slots per CTA for partial tiles
  uint32_t* sk_flags;   // one flag per slot (a tag of `epoch` and the round when valid), followed
                        // at 4 * grid words by one reader count per slot
  uint32_t epoch;       // distinguishes this launch's flags from earlier launches' (1 .. 2^26-1)
  PeerSync peer;        // all zero unless kFlagPeerSync is set
  RoundPlan round_plan; // read when sk_rounds > 1
};

struct KernelVariant {
  int block_m;    // tile rows (128 * cta_group)
  int block_n;    // tile columns
  int rstep;      // k per stage
  int cta_group;  // 1 or 2
  int mode;       // 1 / 3 (fp32 operands: 1xTF32 / 3xTF32), 16 (bf16), 17 (fp16)
  int layout;     // 0 = A[M,K], B[K,N]; 1 = B given as Bt[N,K]; 2 = skinny (roles swapped);
                  // 3 = skinny on the CUDA cores (fp32 FMAs)
  int stages;
  int smem_bytes;
  int tmem_cols;
  int threads;
  int staging_bytes;  // shared memory set aside for the TMA-store output path (0 = kernel lacks it)
  int gave_up_stage;  // 1 = the form of a kernel whose ring is one stage shorter to fit that area
  const void* func;  // kernel symbol, for cudaFuncSetAttribute / occupancy queries
  cudaError_t (*launch)(const GemmArgs& args, int grid, cudaStream_t stream);
};

int variant_count();
const KernelVariant& variant_at(int idx);
// The kernels for 16-bit operands (mode 16 = bf16, 17 = fp16), kept in their own table.
const KernelVariant* variants_16bit(int* n);
// Returns nullptr when no kernel was compiled for the combination.
const KernelVariant* find_variant(int block_m, int block_n, int rstep, int cta_group, int mode,
                                  int layout);
// The form of `kv` with a shorter ring and the staging area of the TMA-store path, if `kv`
// lacks the area and such a form was compiled; else nullptr.
const KernelVariant* find_staged_form(const KernelVariant* kv);
// The kernels with a shorter ring for 16-bit operands, kept beside the 16-bit table.
const KernelVariant* staged_forms_16bit(int* n);

// The CUDA-core kernel for a C of at most 16 rows per pass (layout 3, fp32 FMAs; mode 3 only).
const KernelVariant* simt_skinny_variant();
int skinny_simt_tiles(int M, int N, int* row_groups, int* strips);
int skinny_simt_splits(int M, int N, int K, int sm_count);
size_t skinny_simt_workspace_floats(int M, int N, int splits);
cudaError_t skinny_simt_launch(const float* A, const float* B, float* C, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int splits,
                               float* workspace, int sm_count, cudaStream_t stream);

}  // namespace rb200
