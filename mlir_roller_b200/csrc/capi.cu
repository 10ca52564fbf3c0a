// C ABI of libroller_b200: plans, tensor-map encoding, launch, timing. See include/roller_b200.h
// for the contract of each entry point and the reference interface it stands in for.
#include "../../include/roller_b200.h"

#include <cstdio>
#include <cstring>
#include <new>

#include "gemm_launch.h"

namespace {

using namespace rb200;

thread_local char g_cuda_err[256] = "";

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  cudaGetLastError();  // clear the sticky-free error state
  return ROLLER_ERR_CUDA;
}

#define RB_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e_ = (call);                            \
    if (e_ != cudaSuccess) return cuda_fail(e_, #call); \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library has no link-time
// dependency on libcuda.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// Element types a tensor map can be encoded for.
enum ElemType { kElemF32 = 0, kElemTf32 = 1, kElemBf16 = 2, kElemF16 = 3 };

int elem_bytes_of_mode(int mode) {
  return (mode == ROLLER_MODE_BF16 || mode == ROLLER_MODE_F16) ? 2 : 4;
}

// Row-major matrix `rows x cols` with row stride `ld` elements, loaded in boxes of
// box_rows x box_cols; out-of-range elements read as zero. With kElemTf32 the TMA unit rounds
// every fp32 element to the nearest TF32 value on its way into shared memory (measured on
// B200: 1xTF32 error 6.4e-4 -> 2.4e-4 against truncation by the tensor core, at no cost); the
// 3xTF32 mode needs the raw words and loads them untouched (kElemF32).
int encode_matrix(CUtensorMap* tm, const void* base, long long rows, long long cols, long long ld,
                  int box_cols, int box_rows, CUtensorMapSwizzle swz, ElemType et) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled entry point not found");
    return ROLLER_ERR_CUDA;
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const size_t eb = (et == kElemBf16 || et == kElemF16) ? 2 : 4;
  const CUtensorMapDataType dt = et == kElemBf16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : et == kElemF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : et == kElemTf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32
                                                   : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * eb};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, dt, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "cuTensorMapEncodeTiled failed with CUresult %d",
             static_cast<int>(r));
    return ROLLER_ERR_CUDA;
  }
  return ROLLER_OK;
}

// Copies a rows x cols matrix into a buffer whose rows are a multiple of 16 bytes long, so
// that TMA's 16-byte stride rule holds for operands with odd leading dimensions. HBM-bound:
// one thread moves 16 bytes -- scalar loads (the source rows start anywhere), one 128-bit store
// (the destination rows are aligned); grid.y walks the rows, so no index is ever divided.
template <typename T>
__global__ void pad_rows_kernel(const T* __restrict__ src, long long ld_src,
                                T* __restrict__ dst, long long ld_dst, int rows, int cols) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));   // elements per 128-bit store
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c0 >= cols) return;
#pragma unroll 2
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {
    const T* s = src + static_cast<long long>(r) * ld_src + c0;
    alignas(16) T v[V];
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = (c0 + j < cols) ? s[j] : T(0);
    T* d = dst + static_cast<long long>(r) * ld_dst + c0;
    if (c0 + V <= ld_dst) {
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(v);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j)
        if (c0 + j < cols) d[j] = v[j];
    }
  }
}

// Smallest leading dimension >= x whose rows are a multiple of 16 bytes long.
long long round_up_ld(long long x, int elem_bytes) {
  const long long q = 16 / elem_bytes;
  return (x + q - 1) / q * q;
}

void pad_rows(const void* src, long long ld_src, void* dst, long long ld_dst, int rows, int cols,
              int elem_bytes, int blocks, cudaStream_t st) {
  const int per_thread = 16 / elem_bytes;
  const int threads = 256;
  const int gx = (cols + threads * per_thread - 1) / (threads * per_thread);
  int gy = blocks / gx;                       // about `blocks` CTAs in all
  if (gy < 1) gy = 1;
  if (gy > rows) gy = rows;
  if (gy > 65535) gy = 65535;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), 1);
  if (elem_bytes == 2)
    pad_rows_kernel<uint16_t><<<grid, threads, 0, st>>>(static_cast<const uint16_t*>(src), ld_src,
                                                       static_cast<uint16_t*>(dst), ld_dst, rows, cols);
  else
    pad_rows_kernel<float><<<grid, threads, 0, st>>>(static_cast<const float*>(src), ld_src,
                                                    static_cast<float*>(dst), ld_dst, rows, cols);
}

}  // namespace

struct roller_plan;
static int plan_configure(roller_plan* p);
static cudaError_t bind_variant(roller_plan* p, const KernelVariant* kv);
static int default_unit_kb(const roller_plan* p);

struct roller_plan {
  const KernelVariant* kv;
  int device;
  int sm_count;
  int M, N, K;
  long long lda, ldb, ldc;
  int mode, flags;
  int elem;               // bytes per element of A and B
  int c_elem;             // bytes per element of C
  int layout;             // 0 plain, 1 B given transposed, 2 skinny (roles swapped)
  int tiles_m, tiles_n, grid;
  int chunk_kb;           // accumulation chunk, in k-blocks (one reduce step each)
  int unit_kb;            // unit of the stream-K schedule, in k-blocks (<= chunk_kb)
  int max_clusters;       // co-resident CTA pairs the device reports (cta_group 2 only)
  int max_workers;        // persistent workers (CTAs or CTA pairs) that may run at once
  bool grid_forced;       // grid fixed by roller_b200_gemm_set_grid
  int sk_mode;            // stream-K: -1 = decide per problem, 0 = off, 1 = on whenever possible
  int sk_tiles;           // tiles currently dealt out in k-chunks
  float* sk_ws;           // stream-K partial-tile slots (device), owned
  uint32_t* sk_flags;     // one flag per CTA (device), owned
  int sk_slots;           // CTAs the scratch area was sized for
  uint32_t epoch;         // launch counter for the flags (1 .. 2^26-1)
  int sk_rounds;          // rounds of the progressive schedule in use (1 = plain stream-K)
  int progressive;        // requested rounds of the progressive schedule; 0 = off
  int round_ratio;        // size of a round relative to the previous one, in percent
  rb200::RoundPlan round_plan;  // first tile of every round in use
  long long spin_limit;   // clock cycles a device-side wait may last
  bool overlap_launch;    // launches carry the programmatic-stream-serialization attribute
  bool tma_store;         // C leaves through shared memory and TMA stores
  bool tma_forced;        // ... because the caller asked for it (else: chosen by the library)
  bool coop_fixup;        // progressive schedule: shared tiles are completed by all their workers
  bool drop_publish;      // test aid: partial tiles are never flagged
  bool early_exit;        // CTAs leave once their last tile has been read from shared memory
  bool stage_a, stage_b;  // operands go through a padded copy
  void* ws_a;             // padded copies (device), owned
  void* ws_b;
  long long ws_lda, ws_ldb;
  uint32_t* status;  // device status word, followed by the arrival counter of synced launches; owned
  rb200::PeerSync peer;  // set for the duration of one roller_b200_gemm_run_synced call
  // cached tensor maps for the last (A, B) pointers seen
  const void* map_a_ptr;
  const void* map_b_ptr;
  const void* map_c_ptr;
  CUtensorMap tmA, tmB, tmC;
  // host-buffer path
  void *hd_a, *hd_b, *hd_c;
  cudaEvent_t ev0, ev1;
};

extern "C" {

int roller_b200_device_info(int dev, roller_dev_info* out) {
  if (!out) return ROLLER_ERR_INVALID;
  cudaDeviceProp p;
  RB_CUDA(cudaGetDeviceProperties(&p, dev));
  memset(out, 0, sizeof(*out));
  out->cc_major = p.major;
  out->cc_minor = p.minor;
  out->sm_count = p.multiProcessorCount;
  out->smem_per_block_optin = static_cast<int>(p.sharedMemPerBlockOptin);
  out->smem_per_sm = static_cast<int>(p.sharedMemPerMultiprocessor);
  out->regs_per_sm = p.regsPerMultiprocessor;
  out->l2_bytes = p.l2CacheSize;
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, dev) == cudaSuccess) out->sm_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, dev) == cudaSuccess)
    out->mem_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, dev) == cudaSuccess)
    out->mem_bus_bits = v;
  out->tmem_columns = (p.major == 10) ? 512 : 0;
  out->total_mem = p.totalGlobalMem;
  strncpy(out->name, p.name, sizeof(out->name) - 1);
  return ROLLER_OK;
}

// Index (into the variant table) of the 1xTF32 entry of the idx-th enumerable rTile. The table
// holds the two modes of a tile next to each other; variants for a transposed B share the
// geometry of the plain tiles and are reached through ROLLER_FLAG_B_TRANSPOSED instead.
static int enumerable_variant(int idx) {
  int seen = 0;
  for (int i = 0; i + 1 < variant_count(); i += 2) {
    if (variant_at(i).layout == 1) continue;
    if (seen == idx) return i;
    ++seen;
  }
  return -1;
}

// The tensor-core rTiles come first; the CUDA-core kernel for a C of few rows is the last one.
static int tensor_tile_count() {
  int n = 0;
  while (enumerable_variant(n) >= 0) ++n;
  return n;
}

int roller_b200_kernel_count(void) { return tensor_tile_count() + 1; }

int roller_b200_kernel_desc(int idx, roller_ktile* out) {
  if (!out || idx < 0) return ROLLER_ERR_INVALID;
  if (idx == tensor_tile_count()) {
    const KernelVariant* v = simt_skinny_variant();
    memset(out, 0, sizeof(*out));
    out->block_m = v->block_m;
    out->block_n = v->block_n;
    out->rstep = v->rstep;
    out->cta_group = 1;
    out->stages_3x = v->stages;      // fp32-accurate only: no 1xTF32 and no 16-bit form
    out->smem_3x = v->smem_bytes;
    out->threads_3x = v->threads;
    out->layout = v->layout;
    return ROLLER_OK;
  }
  const int vi = enumerable_variant(idx);
  if (vi < 0) return ROLLER_ERR_INVALID;
  const KernelVariant& v1 = variant_at(vi);
  const KernelVariant& v3 = variant_at(vi + 1);
  out->block_m = v1.block_m;
  out->block_n = v1.block_n;
  out->rstep = v1.rstep;
  out->cta_group = v1.cta_group;
  out->stages_1x = v1.stages;
  out->stages_3x = v3.stages;
  out->smem_1x = v1.smem_bytes;
  out->smem_3x = v3.smem_bytes;
  out->tmem_cols = v1.tmem_cols;
  out->threads_1x = v1.threads;
  out->threads_3x = v3.threads;
  out->layout = v1.layout;
  const KernelVariant* v16 = find_variant(v1.block_m, v1.block_n, 2 * v1.rstep, v1.cta_group,
                                          ROLLER_MODE_BF16, v1.layout);
  out->rstep_16 = v16 ? v16->rstep : 0;
  out->stages_16 = v16 ? v16->stages : 0;
  out->smem_16 = v16 ? v16->smem_bytes : 0;
  return ROLLER_OK;
}

int roller_b200_gemm_create(const roller_ktile* tile, int M, int N, int K, int lda, int ldb, int ldc,
                            int mode, int flags, roller_plan** out) {
  if (!tile || !out) return ROLLER_ERR_INVALID;
  *out = nullptr;
  if (flags & ~(ROLLER_FLAG_ACCUMULATE | ROLLER_FLAG_B_TRANSPOSED | ROLLER_FLAG_C_16BIT))
    return ROLLER_ERR_INVALID;
  const bool b_transposed = (flags & ROLLER_FLAG_B_TRANSPOSED) != 0;
  if (M <= 0 || N <= 0 || K <= 0 || lda < K || ldb < (b_transposed ? K : N) || ldc < N)
    return ROLLER_ERR_INVALID;
  if (mode != ROLLER_MODE_1XTF32 && mode != ROLLER_MODE_3XTF32 && mode != ROLLER_MODE_BF16 &&
      mode != ROLLER_MODE_F16)
    return ROLLER_ERR_INVALID;
  const int elem = elem_bytes_of_mode(mode);
  if ((flags & ROLLER_FLAG_C_16BIT) && elem != 2) return ROLLER_ERR_INVALID;
  if (tile->layout != 0 && tile->layout != 2 && tile->layout != 3) return ROLLER_ERR_INVALID;
  if (b_transposed && tile->layout != 0) return ROLLER_ERR_UNSUPPORTED;
  // the CUDA-core kernel computes in plain fp32: it serves the fp32-accurate mode, C = A @ B
  if (tile->layout == 3 && (mode != ROLLER_MODE_3XTF32 || flags != 0)) return ROLLER_ERR_UNSUPPORTED;
  const int layout = b_transposed ? 1 : tile->layout;
  // a 16-bit kernel reduces the same 128 bytes of k per step: twice the elements
  const KernelVariant* kv = find_variant(tile->block_m, tile->block_n,
                                         tile->rstep * (4 / elem), tile->cta_group, mode, layout);
  if (!kv) return ROLLER_ERR_UNSUPPORTED;

  int dev = 0;
  RB_CUDA(cudaGetDevice(&dev));
  cudaDeviceProp prop;
  RB_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10) return ROLLER_ERR_DEVICE;
  if (static_cast<int>(prop.sharedMemPerBlockOptin) < kv->smem_bytes) return ROLLER_ERR_DEVICE;

  roller_plan* p = new (std::nothrow) roller_plan();
  if (!p) return ROLLER_ERR_NOMEM;
  memset(p, 0, sizeof(*p));
  p->kv = kv;
  p->device = dev;
  p->sm_count = prop.multiProcessorCount;
  p->M = M; p->N = N; p->K = K;
  p->lda = lda; p->ldb = ldb; p->ldc = ldc;
  p->mode = mode;
  p->elem = elem;
  p->c_elem = (flags & ROLLER_FLAG_C_16BIT) ? 2 : 4;
  p->flags = flags;
  p->layout = layout;
  if (layout == 3) {
    skinny_simt_tiles(M, N, &p->tiles_m, &p->tiles_n);
  } else if (layout == 2) {
    // the kernel works on C^T: its tile rows (128) run along N, its tile columns along M
    p->tiles_m = (N + kv->block_n - 1) / kv->block_n;
    p->tiles_n = (M + kv->block_m - 1) / kv->block_m;
  } else {
    p->tiles_m = (M + kv->block_m - 1) / kv->block_m;
    p->tiles_n = (N + kv->block_n - 1) / kv->block_n;
  }
  p->max_workers = p->sm_count / kv->cta_group;
  p->sk_mode = -1;
  p->epoch = 0;
  p->sk_rounds = 1;
  p->spin_limit = kSpinLimitCycles;
  p->overlap_launch = true;
  p->coop_fixup = true;
  // Where the kernel has the staging area and C qualifies, C leaves through TMA stores: measured
  // 3-6 % faster than the accumulate warps' own stores on every README shape (whole 128-byte
  // lines leave the SM, and the warps are back at the next tile sooner).
  p->tma_store = false;   // decided below, once the kernel is bound
  // 3xTF32 drains the TMEM accumulator every 128 k (see the kernel header); 1xTF32 is
  // dominated by the 10-bit input mantissa, so one chunk spans the whole reduction.
  const int num_kb = (K + kv->rstep - 1) / kv->rstep;
  p->chunk_kb = (mode == ROLLER_MODE_3XTF32) ? 4 : num_kb;
  // 16-bit products are exact, so the accumulator's rounding is the whole error. Measured on
  // B200 (uniform inputs): 2.3e-6 of max|C| with a drain every 2048 k at any K, 1.1e-5 at
  // K = 8192 without drains; shorter chunks cost throughput (1024 k: -6 %, 512 k: -13 %).
  if (elem == 2 && num_kb > 32) p->chunk_kb = 32;
  // A skinny problem streams B once and is HBM-bound: it needs every SM pulling data, which
  // only a split along K provides, so 1xTF32 gets chunks too (512 k).
  if (layout == 2 && mode != ROLLER_MODE_3XTF32 && num_kb > 16) p->chunk_kb = 16;
  p->unit_kb = default_unit_kb(p);
  // (the CUDA-core kernel loads with plain instructions and takes any alignment)
  p->stage_a = layout != 3 && (static_cast<long long>(lda) * elem % 16) != 0;
  p->stage_b = layout != 3 && (static_cast<long long>(ldb) * elem % 16) != 0;

  // Whether C can leave through TMA stores at all (the base address is checked per launch).
  const bool c_fits_tma = layout != 2 && p->c_elem == 4 && !(flags & ROLLER_FLAG_ACCUMULATE) &&
                          ldc % 4 == 0;
  // A kernel whose ring fills shared memory also exists with one stage less and the staging
  // area of that path; for the pair tile that form is the faster one up to K = 4096 (see
  // GemmCfg; the single-CTA 128 x 128 tile gains nothing from it and switches only on request).
  // An fp32 C whose rows are not 16-byte aligned is written through the same staging area (see
  // kFlagSmemStore): the form with the area then pays at any K.
  const bool c_ragged = layout == 0 || layout == 1 ? (p->c_elem == 4 && ldc % 4 != 0) : false;
  if ((c_fits_tma && K <= 4096 && kv->cta_group == 2) || (c_ragged && kv->staging_bytes == 0)) {
    const KernelVariant* staged = find_staged_form(kv);
    if (staged && static_cast<int>(prop.sharedMemPerBlockOptin) >= staged->smem_bytes) kv = staged;
  }
  cudaError_t e = layout == 3 ? cudaSuccess : bind_variant(p, kv);
  p->tma_store = p->kv->staging_bytes > 0 && c_fits_tma;
  if (e == cudaSuccess) e = cudaMalloc(&p->status, 2 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(p->status, 0, 2 * sizeof(uint32_t));
  if (e == cudaSuccess && p->stage_a) {
    p->ws_lda = round_up_ld(K, elem);
    e = cudaMalloc(&p->ws_a, static_cast<size_t>(elem) * p->ws_lda * M);
  }
  if (e == cudaSuccess && p->stage_b) {
    p->ws_ldb = round_up_ld(b_transposed ? K : N, elem);
    e = cudaMalloc(&p->ws_b, static_cast<size_t>(elem) * p->ws_ldb * (b_transposed ? N : K));
  }
  if (e == cudaSuccess) e = cudaEventCreate(&p->ev0);
  if (e == cudaSuccess) e = cudaEventCreate(&p->ev1);
  if (e != cudaSuccess) {
    int rc = (e == cudaErrorMemoryAllocation) ? ROLLER_ERR_NOMEM : cuda_fail(e, "plan setup");
    cudaGetLastError();
    roller_b200_gemm_destroy(p);
    return rc;
  }
  int rc = plan_configure(p);
  if (rc != ROLLER_OK) {
    roller_b200_gemm_destroy(p);
    return rc;
  }
  *out = p;
  return ROLLER_OK;
}

int roller_b200_gemm_run(roller_plan* p, const void* A, const void* B, void* C, void* stream) {
  if (!p || !A || !B || !C) return ROLLER_ERR_INVALID;
  // a plan's workspaces, tensor maps and status word live on the device it was created on
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess || cur != p->device) return ROLLER_ERR_DEVICE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const KernelVariant* kv = p->kv;
  if (p->layout == 3) {
    RB_CUDA(skinny_simt_launch(static_cast<const float*>(A), static_cast<const float*>(B),
                               static_cast<float*>(C), p->M, p->N, p->K, p->lda, p->ldb, p->ldc,
                               p->sk_rounds, p->sk_ws, p->sm_count, st));
    return ROLLER_OK;
  }

  // Operands that break TMA's rules (row stride or base not a multiple of 16 bytes) are staged
  // through a padded copy; the base-alignment case needs a workspace made on demand at create
  // time, so an unaligned base with an aligned stride is rejected here.
  const void* a_src = A;
  const void* b_src = B;
  long long lda = p->lda, ldb = p->ldb;
  // every argument is checked before anything is enqueued
  if (!p->stage_a && (reinterpret_cast<uintptr_t>(A) & 15)) return ROLLER_ERR_INVALID;
  if (!p->stage_b && (reinterpret_cast<uintptr_t>(B) & 15)) return ROLLER_ERR_INVALID;
  const bool c_aligned = (reinterpret_cast<uintptr_t>(C) & 15) == 0;
  if (p->tma_store && p->tma_forced && !c_aligned) return ROLLER_ERR_INVALID;
  const bool tma_store = p->tma_store && c_aligned;
  const bool peer_sync = p->peer.go_flag || p->peer.arrive_flag;
  if (peer_sync && !tma_store) return ROLLER_ERR_UNSUPPORTED;
  if (p->stage_a) {
    pad_rows(A, p->lda, p->ws_a, p->ws_lda, p->M, p->K, p->elem, p->sm_count * 8, st);
    a_src = p->ws_a;
    lda = p->ws_lda;
  }
  if (p->stage_b) {
    if (p->layout == 1)
      pad_rows(B, p->ldb, p->ws_b, p->ws_ldb, p->N, p->K, p->elem, p->sm_count * 8, st);
    else
      pad_rows(B, p->ldb, p->ws_b, p->ws_ldb, p->K, p->N, p->elem, p->sm_count * 8, st);
    b_src = p->ws_b;
    ldb = p->ws_ldb;
  }
  if (p->stage_a || p->stage_b) RB_CUDA(cudaGetLastError());

  // Which matrix feeds which MMA operand depends on the layout (see the kernel header).
  if (a_src != p->map_a_ptr || b_src != p->map_b_ptr) {
    int rc;
    const int bnl = (p->layout == 2 ? kv->block_m : kv->block_n) / kv->cta_group;
    const ElemType et = p->mode == ROLLER_MODE_1XTF32 ? kElemTf32
                        : p->mode == ROLLER_MODE_BF16 ? kElemBf16
                        : p->mode == ROLLER_MODE_F16  ? kElemF16
                                                      : kElemF32;
    // every box row is 128 bytes: `bk` elements, which is also the reduce step; an operand
    // that is contiguous along m/n is fetched in square boxes (fp32: 32-byte swizzle chunks)
    const int bk = 128 / p->elem;
    const CUtensorMapSwizzle swz_mn =
        p->elem == 4 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    if (p->layout == 2) {
      rc = encode_matrix(&p->tmA, b_src, p->K, p->N, ldb, bk, bk, swz_mn, et);
      if (rc == ROLLER_OK)
        rc = encode_matrix(&p->tmB, a_src, p->M, p->K, lda, bk, bnl, CU_TENSOR_MAP_SWIZZLE_128B, et);
    } else {
      rc = encode_matrix(&p->tmA, a_src, p->M, p->K, lda, bk, 128, CU_TENSOR_MAP_SWIZZLE_128B, et);
      if (rc == ROLLER_OK && p->layout == 1)
        rc = encode_matrix(&p->tmB, b_src, p->N, p->K, ldb, bk, bnl, CU_TENSOR_MAP_SWIZZLE_128B, et);
      else if (rc == ROLLER_OK)
        rc = encode_matrix(&p->tmB, b_src, p->K, p->N, ldb, bk, bk, swz_mn, et);
    }
    if (rc != ROLLER_OK) return rc;
    p->map_a_ptr = a_src;
    p->map_b_ptr = b_src;
  }
  if (tma_store && C != p->map_c_ptr) {
    // C as a store destination: boxes of 32 x 32 fp32 under the 128-byte swizzle. C may be
    // another GPU's memory mapped into this process; the map is never used for a load.
    int rc = encode_matrix(&p->tmC, C, p->M, p->N, p->ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B,
                           kElemF32);
    if (rc != ROLLER_OK) return rc;
    p->map_c_ptr = C;
  }

  GemmArgs args;
  args.tmA = p->tmA;
  args.tmB = p->tmB;
  if (tma_store) args.tmC = p->tmC; else memset(&args.tmC, 0, sizeof(args.tmC));
  args.C = static_cast<float*>(C);
  args.M = (p->layout == 2) ? p->N : p->M;
  args.N = (p->layout == 2) ? p->M : p->N;
  args.K = p->K;
  args.ldc = p->ldc;
  args.tiles_m = p->tiles_m;
  args.tiles_n = p->tiles_n;
  args.chunk_kb = p->unit_kb;
  args.acc_kb = p->chunk_kb;
  args.flags = (p->flags & ROLLER_FLAG_ACCUMULATE) ? kFlagAccumulate : 0;
  if ((p->ldc * p->c_elem % 16) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0)
    args.flags |= kFlagVecStore;
  if (p->c_elem == 2) args.flags |= kFlagC16;
  if (tma_store) args.flags |= kFlagTmaStore;
  // rows of an fp32 C that start anywhere: coalesced stores through the staging area
  if (!tma_store && kv->staging_bytes > 0 && p->c_elem == 4 && p->layout != 2 &&
      !(args.flags & kFlagVecStore))
    args.flags |= kFlagSmemStore;
  // In the progressive schedule tiles are shared on purpose. With this flag the kernel lets
  // all workers of a tile complete it together in the rounds where a tile is shared by three
  // workers or more; in the others the worker holding the end of the reduction does it alone.
  if (tma_store && p->progressive != 0 && p->sk_tiles > 0 && p->coop_fixup)
    args.flags |= kFlagCoopFixup;
  if (p->drop_publish) args.flags |= kFlagDropPublish;
  if (p->early_exit) args.flags |= kFlagEarlyExit;
  args.round_plan = p->round_plan;
  args.peer = p->peer;
  if (peer_sync) {
    args.flags |= kFlagPeerSync;
    args.peer.arrive_count = p->status + 1;
  }
  args.status = p->status;
  args.spin_limit = p->spin_limit;
  args.serialize_programmatically = p->overlap_launch;
  args.sk_tiles = p->sk_tiles;
  args.sk_rounds = p->sk_rounds;
  args.sk_ws = p->sk_ws;
  args.sk_flags = p->sk_flags;
  p->epoch = p->epoch % 0x3FFFFFFu + 1;   // never zero: zero in a flag means "slot free"
  args.epoch = p->epoch;
  RB_CUDA(kv->launch(args, p->grid, st));
  return ROLLER_OK;
}

int roller_b200_gemm_run_synced(roller_plan* p, const void* A, const void* B, void* C,
                                const uint32_t* go_flag, uint32_t go_value, uint32_t* arrive_flag,
                                uint32_t arrive_value, void* stream) {
  if (!p) return ROLLER_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(go_flag) & 3) || (reinterpret_cast<uintptr_t>(arrive_flag) & 3))
    return ROLLER_ERR_INVALID;
  // the kernel's own hand-shake exists on the TMA-store output path only
  if (p->layout == 3 || !p->tma_store) return ROLLER_ERR_UNSUPPORTED;
  p->peer.go_flag = go_flag;
  p->peer.go_value = go_value;
  p->peer.arrive_flag = arrive_flag;
  p->peer.arrive_value = arrive_value;
  const int rc = roller_b200_gemm_run(p, A, B, C, stream);
  p->peer = rb200::PeerSync{};
  return rc;
}

int roller_b200_gemm_time(roller_plan* p, const void* A, const void* B, void* C, void* stream,
                          int warmup, int iters, float* ms_per_iter) {
  if (!p || !ms_per_iter || iters <= 0 || warmup < 0) return ROLLER_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int i = 0; i < warmup; ++i) {
    int rc = roller_b200_gemm_run(p, A, B, C, stream);
    if (rc != ROLLER_OK) return rc;
  }
  RB_CUDA(cudaStreamSynchronize(st));
  RB_CUDA(cudaEventRecord(p->ev0, st));
  for (int i = 0; i < iters; ++i) {
    int rc = roller_b200_gemm_run(p, A, B, C, stream);
    if (rc != ROLLER_OK) return rc;
  }
  RB_CUDA(cudaEventRecord(p->ev1, st));
  RB_CUDA(cudaEventSynchronize(p->ev1));
  float ms = 0.f;
  RB_CUDA(cudaEventElapsedTime(&ms, p->ev0, p->ev1));
  *ms_per_iter = ms / static_cast<float>(iters);
  return ROLLER_OK;
}

int roller_b200_gemm_host_async(roller_plan* p, const void* hA, const void* hB, void* hC,
                                void* stream) {
  if (!p || !hA || !hB || !hC) return ROLLER_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t a_bytes = static_cast<size_t>(p->elem) * static_cast<size_t>(p->lda) * p->M;
  const size_t b_bytes =
      static_cast<size_t>(p->elem) * static_cast<size_t>(p->ldb) * (p->layout == 1 ? p->N : p->K);
  const size_t c_bytes = static_cast<size_t>(p->c_elem) * static_cast<size_t>(p->ldc) * p->M;
  if (!p->hd_a) {
    cudaError_t e = cudaMalloc(&p->hd_a, a_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->hd_b, b_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->hd_c, c_bytes);
    if (e != cudaSuccess) {
      cudaFree(p->hd_a); cudaFree(p->hd_b); cudaFree(p->hd_c);
      p->hd_a = p->hd_b = p->hd_c = nullptr;
      cudaGetLastError();
      return ROLLER_ERR_NOMEM;
    }
  }
  RB_CUDA(cudaMemcpyAsync(p->hd_a, hA, a_bytes, cudaMemcpyHostToDevice, st));
  RB_CUDA(cudaMemcpyAsync(p->hd_b, hB, b_bytes, cudaMemcpyHostToDevice, st));
  if (p->flags & ROLLER_FLAG_ACCUMULATE)
    RB_CUDA(cudaMemcpyAsync(p->hd_c, hC, c_bytes, cudaMemcpyHostToDevice, st));
  int rc = roller_b200_gemm_run(p, p->hd_a, p->hd_b, p->hd_c, stream);
  if (rc != ROLLER_OK) return rc;
  RB_CUDA(cudaMemcpyAsync(hC, p->hd_c, c_bytes, cudaMemcpyDeviceToHost, st));
  return ROLLER_OK;
}

int roller_b200_gemm_host(roller_plan* p, const void* hA, const void* hB, void* hC, void* stream) {
  int rc = roller_b200_gemm_host_async(p, hA, hB, hC, stream);
  if (rc != ROLLER_OK) return rc;
  RB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return ROLLER_OK;
}

int roller_b200_copy_block_async(float* dst, long long dst_ld, const float* src, long long src_ld,
                                 long long rows, long long cols, void* stream) {
  if (rows < 0 || cols < 0 || dst_ld < cols || src_ld < cols) return ROLLER_ERR_INVALID;
  if (rows == 0 || cols == 0) return ROLLER_OK;
  if (!dst || !src) return ROLLER_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t width = sizeof(float) * static_cast<size_t>(cols);
  if (dst_ld == cols && src_ld == cols) {
    RB_CUDA(cudaMemcpyAsync(dst, src, width * static_cast<size_t>(rows), cudaMemcpyDefault, st));
  } else {
    RB_CUDA(cudaMemcpy2DAsync(dst, sizeof(float) * static_cast<size_t>(dst_ld), src,
                              sizeof(float) * static_cast<size_t>(src_ld), width,
                              static_cast<size_t>(rows), cudaMemcpyDefault, st));
  }
  return ROLLER_OK;
}

int roller_b200_gemm_launch_info(const roller_plan* p, int* grid, int* block, int* smem_bytes,
                                 int* tiles_m, int* tiles_n, int* max_clusters) {
  if (!p) return ROLLER_ERR_INVALID;
  if (grid) *grid = p->grid;
  if (block) *block = p->kv->threads;
  if (smem_bytes) *smem_bytes = p->kv->smem_bytes;
  if (tiles_m) *tiles_m = p->tiles_m;
  if (tiles_n) *tiles_n = p->tiles_n;
  if (max_clusters) *max_clusters = p->max_clusters;
  return ROLLER_OK;
}

int roller_b200_gemm_schedule_info(const roller_plan* p, int* sk_tiles, int* rounds, int* unit_kb,
                                   int* chunk_kb) {
  if (!p) return ROLLER_ERR_INVALID;
  if (sk_tiles) *sk_tiles = p->sk_tiles;
  if (rounds) *rounds = p->sk_rounds;
  if (unit_kb) *unit_kb = p->unit_kb;
  if (chunk_kb) *chunk_kb = p->chunk_kb;
  return ROLLER_OK;
}

int roller_b200_gemm_round_tiles(const roller_plan* p, int* tile_begin, int capacity) {
  if (!p || !tile_begin || capacity < p->sk_rounds + 1) return ROLLER_ERR_INVALID;
  if (p->layout == 3) return ROLLER_ERR_UNSUPPORTED;
  for (int r = 0; r <= p->sk_rounds; ++r)
    tile_begin[r] = p->sk_rounds > 1 ? p->round_plan.tile_begin[r] : (r == 0 ? 0 : p->sk_tiles);
  return ROLLER_OK;
}

int roller_b200_gemm_set_chunk(roller_plan* p, int k_elems) {
  if (!p || k_elems < 0) return ROLLER_ERR_INVALID;
  if (p->layout == 3) return ROLLER_OK;   // fp32 FMAs: there is no accumulator to drain
  const int num_kb = (p->K + p->kv->rstep - 1) / p->kv->rstep;
  int kb = (k_elems == 0) ? num_kb : (k_elems + p->kv->rstep - 1) / p->kv->rstep;
  if (kb < 1) kb = 1;
  if (kb > num_kb) kb = num_kb;
  p->chunk_kb = kb;
  p->unit_kb = default_unit_kb(p);
  return plan_configure(p);
}

int roller_b200_gemm_set_grid(roller_plan* p, int ctas) {
  if (!p || ctas <= 0 || ctas % p->kv->cta_group != 0) return ROLLER_ERR_INVALID;
  if (p->layout == 3) return ROLLER_ERR_UNSUPPORTED;
  const long long tiles = static_cast<long long>(p->tiles_m) * p->tiles_n;
  if (ctas / p->kv->cta_group > p->max_workers) return ROLLER_ERR_INVALID;
  if (ctas / p->kv->cta_group > tiles * ((p->K + p->kv->rstep - 1) / p->kv->rstep))
    return ROLLER_ERR_INVALID;
  p->grid = ctas;
  p->grid_forced = true;
  return plan_configure(p);
}

int roller_b200_gemm_set_stream_k(roller_plan* p, int mode) {
  if (!p || mode < -1 || mode > 1) return ROLLER_ERR_INVALID;
  if (p->layout == 3) return ROLLER_OK;   // its split along K is fixed and always reproducible
  p->sk_mode = mode;
  return plan_configure(p);
}

int roller_b200_last_status(roller_plan* p, uint32_t* device_status) {
  if (!p) return ROLLER_ERR_INVALID;
  uint32_t h = 0;
  RB_CUDA(cudaDeviceSynchronize());
  RB_CUDA(cudaMemcpy(&h, p->status, sizeof(h), cudaMemcpyDeviceToHost));
  if (device_status) *device_status = h;
  if (h != 0) {
    // Read and clear: the failed launch has been reported, later launches start clean. The
    // stream-K flags of a launch that gave up may be left raised, so they are reset as well.
    RB_CUDA(cudaMemset(p->status, 0, 2 * sizeof(uint32_t)));   // (with the arrival counter)
    if (p->sk_flags) RB_CUDA(cudaMemset(p->sk_flags, 0, sizeof(uint32_t) * p->sk_slots * 2));
  }
  return h == 0 ? ROLLER_OK : ROLLER_ERR_TIMEOUT;
}

int roller_b200_gemm_set_option(roller_plan* p, int option, long long value) {
  if (!p) return ROLLER_ERR_INVALID;
  switch (option) {
    case ROLLER_OPT_WAIT_LIMIT_CYCLES:
      if (value < 0) return ROLLER_ERR_INVALID;
      p->spin_limit = value == 0 ? kSpinLimitCycles : value;
      return ROLLER_OK;
    case ROLLER_OPT_OVERLAP_LAUNCH:
      p->overlap_launch = value != 0;
      return ROLLER_OK;
    case ROLLER_OPT_TMA_STORE:
      if (value != 0 && p->layout == 3) return ROLLER_ERR_UNSUPPORTED;
      if (value != 0) {
        if (p->layout == 2 || p->c_elem != 4 || (p->flags & ROLLER_FLAG_ACCUMULATE))
          return ROLLER_ERR_UNSUPPORTED;
        if (p->ldc % 4 != 0) return ROLLER_ERR_INVALID;   // TMA needs 16-byte row strides
        if (p->kv->staging_bytes == 0) {
          // the form of the kernel with a shorter ring has the staging area
          const KernelVariant* staged = find_staged_form(p->kv);
          if (!staged) return ROLLER_ERR_UNSUPPORTED;
          if (bind_variant(p, staged) != cudaSuccess) return cuda_fail(cudaGetLastError(), "bind kernel");
          int rc = plan_configure(p);
          if (rc != ROLLER_OK) return rc;
        }
      }
      p->tma_store = value != 0;
      p->tma_forced = value != 0;
      p->map_c_ptr = nullptr;
      return ROLLER_OK;
    case ROLLER_OPT_ROUND_RATIO:
      if (value < 25 || value > 400) return ROLLER_ERR_INVALID;
      p->round_ratio = static_cast<int>(value);
      return plan_configure(p);
    case ROLLER_OPT_PROGRESSIVE_ROUNDS:
      if (value < -1 || value > kMaxRounds) return ROLLER_ERR_INVALID;
      if (value != 0 && ((p->flags & ROLLER_FLAG_ACCUMULATE) || p->layout == 3))
        return ROLLER_ERR_UNSUPPORTED;
      p->progressive = static_cast<int>(value);
      return plan_configure(p);
    case ROLLER_OPT_EARLY_EXIT:
      p->early_exit = value != 0;
      return ROLLER_OK;
    case ROLLER_OPT_COOPERATIVE_FIXUP:
      p->coop_fixup = value != 0;
      return ROLLER_OK;
    case ROLLER_OPT_TEST_DROP_PUBLISH:
      p->drop_publish = value != 0;
      return ROLLER_OK;
    default:
      return ROLLER_ERR_INVALID;
  }
}

int roller_b200_gemm_destroy(roller_plan* p) {
  if (!p) return ROLLER_OK;
  cudaFree(p->ws_a);
  cudaFree(p->ws_b);
  cudaFree(p->status);
  cudaFree(p->sk_ws);
  cudaFree(p->sk_flags);
  cudaFree(p->hd_a);
  cudaFree(p->hd_b);
  cudaFree(p->hd_c);
  if (p->ev0) cudaEventDestroy(p->ev0);
  if (p->ev1) cudaEventDestroy(p->ev1);
  cudaGetLastError();
  delete p;
  return ROLLER_OK;
}

const char* roller_b200_strerror(int status) {
  switch (status) {
    case ROLLER_OK: return "ok";
    case ROLLER_ERR_INVALID: return "invalid argument";
    case ROLLER_ERR_UNSUPPORTED: return "no compiled kernel for this rTile and mode";
    case ROLLER_ERR_CUDA: return "CUDA call failed";
    case ROLLER_ERR_DEVICE: return "current device is not an sm_100 GPU with enough shared memory, or not the device the plan was created on";
    case ROLLER_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case ROLLER_ERR_NOMEM: return "device memory allocation failed";
    case ROLLER_ERR_TOO_LARGE: return "problem exceeds the capacity of this entry point";
    default: return "unknown status";
  }
}

const char* roller_b200_last_cuda_error(void) { return g_cuda_err; }

}  // extern "C"

// Binds the plan to one compiled kernel: raises its shared-memory limit and asks how many of its
// CTA pairs the device can hold at once (a persistent grid must be co-resident).
static cudaError_t bind_variant(roller_plan* p, const KernelVariant* kv) {
  p->kv = kv;
  p->max_workers = p->sm_count / kv->cta_group;
  p->max_clusters = 0;
  cudaError_t e = cudaFuncSetAttribute(kv->func, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kv->smem_bytes);
  if (e == cudaSuccess && kv->cta_group == 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p->sm_count), 1, 1);
    cfg.blockDim = dim3(static_cast<unsigned>(kv->threads), 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(kv->smem_bytes);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kv->func, &cfg);
    if (e == cudaSuccess) {
      p->max_clusters = n;
      if (n > 0 && p->max_workers > n) p->max_workers = n;
    }
  }
  return e;
}

// Chooses the persistent grid and the stream-K split for the plan's current settings, and makes
// sure the stream-K scratch area exists when it is needed. Never called from the run path.
//
// With T tiles on W workers the round-robin schedule takes ceil(T / W) tile-times. Dealing the
// r = T mod W leftover tiles out in k-chunks instead takes floor(T / W) tile-times plus
// ceil(r * chunks_per_tile / W) chunk-times, at the price of one partial-tile exchange per
// worker. That exchange is hidden behind the whole tiles that follow (4096^3: -11 %,
// 2048x8192x8192: -15 %) but exposed when there are fewer tiles than workers, where it costs
// about as much as three 128-deep chunks (64 tiles on 74 CTA pairs: +6 % at K = 2048, -4 % at
// K = 4096 and 8192, -5 % at K = 16384; 48 tiles at K = 8192: -22 %). So the split schedule is
// charged one chunk (whole tiles follow) or three (they do not) and used when it is still at
// least 3 % shorter.
// 3xTF32 drains every chunk for accuracy and deals leftover tiles out in the same pieces. The
// other modes drain rarely (or never), so their schedule gets a unit of its own: 8 k-blocks,
// fine enough to even out a last wave, and never longer than the accumulation chunk.
static int default_unit_kb(const roller_plan* p) {
  if (p->mode == ROLLER_MODE_3XTF32 || p->layout == 2) return p->chunk_kb;
  return p->chunk_kb < 8 ? p->chunk_kb : 8;
}

static int plan_configure(roller_plan* p) {
  const KernelVariant* kv = p->kv;
  if (p->layout == 3) {
    // CUDA-core kernel: strips x K-splits x row groups of CTAs; the partial results of the
    // splits go through a workspace and are added by a second kernel
    const int splits = skinny_simt_splits(p->M, p->N, p->K, p->sm_count);
    p->sk_tiles = 0;
    p->sk_rounds = splits;
    p->grid = p->tiles_m * p->tiles_n * splits;
    const size_t need = skinny_simt_workspace_floats(p->M, p->N, splits);
    if (need && !p->sk_ws) {
      if (cudaMalloc(&p->sk_ws, need * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        return ROLLER_ERR_NOMEM;
      }
    }
    return ROLLER_OK;
  }
  const long long tiles = static_cast<long long>(p->tiles_m) * p->tiles_n;
  const int num_kb = (p->K + kv->rstep - 1) / kv->rstep;
  const int cpt = (num_kb + p->unit_kb - 1) / p->unit_kb;
  int workers = p->grid_forced ? p->grid / kv->cta_group : p->max_workers;
  if (workers < 1) workers = 1;

  int sk_tiles = 0;
  int rounds = 1;
  const long long r = tiles % workers;
  if (p->progressive != 0 && cpt > 1 && tiles * cpt < (1ll << 31)) {
    // Progressive schedule: every tile is cut along K and the tiles are worked through in
    // groups, so that finished tiles appear at a steady rate. The number of rounds must
    // divide the tile count (no tile may straddle two rounds): the largest divisor not above
    // the request is taken. Left to the library (-1), a round holds about as many tiles as
    // there are workers, so that a tile is shared by little more than one worker: the worker
    // completing a tile adds the others' partial sums one after the other, and with more of
    // them the exchange no longer hides behind the two accumulator buffers (measured on B200,
    // 256 x 256 pair tile, 3xTF32, against whole tiles: shared by 1.2 workers 0-4 % slower, by
    // 2.3 workers 5-15 %, by 4.6 workers 35-45 %). Two rounds at least, or nothing would leave
    // early.
    long long want = p->progressive;
    if (want < 0) {
      want = (tiles * 5) / (4ll * workers);        // a tile shared by about 1.2 workers: free
      if (want < 2 && tiles >= workers / 4) want = 2;   // but at least two rounds
      // Less than one wave of tiles: without rounds everything would leave at the very end.
      // Four rounds (tiles shared by four to five workers, completed cooperatively) cost a
      // quarter more time and put three quarters of the output on its way early.
      if (tiles <= workers && tiles >= workers / 2) want = 4;
    }
    if (want > kMaxRounds) want = kMaxRounds;
    if (want > tiles) want = tiles;
    if (want < 1) want = 1;
    rounds = static_cast<int>(want);
    sk_tiles = static_cast<int>(tiles);
    // Equal rounds of fewer tiles than workers: with a worker count that the round's tiles
    // divide, every tile is shared by the same number of workers and every worker publishes
    // exactly one partial per round. Giving up to a sixth of the workers for that pays in the
    // modes whose main loop is short against the exchange (64 tiles on 64 instead of 74 CTA
    // pairs, timed alternately in one process: 1xTF32 in 4 rounds 108 -> 80 us, in 2 rounds
    // 68 -> 62 us; 3xTF32 unchanged within a per cent).
    if (!p->grid_forced && (p->round_ratio == 0 || p->round_ratio == 100) && tiles % rounds == 0) {
      const long long per_round = tiles / rounds;
      if (per_round < workers) {
        const long long even = workers / per_round * per_round;
        if (even * 6 >= static_cast<long long>(workers) * 5) workers = static_cast<int>(even);
      }
    }
  } else if (p->sk_mode != 0 && r != 0 && cpt > 1 && !(p->flags & ROLLER_FLAG_ACCUMULATE)) {
    const long long full = tiles / workers;
    const long long dp_time = (full + 1) * cpt;
    // Cost of handing partial tiles from worker to worker through global memory, in units:
    // one unit, three when no whole tile follows to hide the wait, for 3xTF32 (4.4 us per
    // unit); 24 k-blocks, or 72, for the faster modes (fitted to measurements: 4096^3 and
    // 2048 x 4096 x 4096 gain 7-10 % in 1xTF32, 2048^3 would lose 9 %).
    const long long per_exchange = (p->mode == ROLLER_MODE_3XTF32) ? 1 : (24 + p->unit_kb - 1) / p->unit_kb;
    const long long exchange = per_exchange * (full >= 1 ? 1 : 3);
    const long long sk_time = full * cpt + (r * cpt + workers - 1) / workers + exchange;
    // (the skinny layout is HBM-bound: it always splits, to put every SM to work on the stream)
    if (p->sk_mode == 1 || p->layout == 2 || (dp_time - sk_time) * 100 >= 3 * dp_time)
      sk_tiles = static_cast<int>(r);
  }
  if (!p->grid_forced) {
    const long long units = sk_tiles ? static_cast<long long>(sk_tiles) * cpt + (tiles - sk_tiles)
                                     : tiles;
    long long w = units < workers ? units : workers;
    if (sk_tiles && tiles >= workers) w = workers;
    p->grid = static_cast<int>(w) * kv->cta_group;
  }
  p->sk_tiles = sk_tiles;
  p->sk_rounds = rounds;
  // The rounds' shares of the tiles: a geometric sequence with the plan's ratio, every round at
  // least one tile (the boundaries are rounded cumulative shares, pushed apart where needed).
  {
    const double ratio = p->round_ratio > 0 ? p->round_ratio / 100.0 : 1.0;
    double total = 0.0, term = 1.0;
    for (int r = 0; r < rounds; ++r, term *= ratio) total += term;
    double cum = 0.0;
    term = 1.0;
    p->round_plan.tile_begin[0] = 0;
    for (int r = 1; r <= rounds; ++r, term *= ratio) {
      cum += term;
      long long b = static_cast<long long>(cum / total * sk_tiles + 0.5);
      const long long lo = p->round_plan.tile_begin[r - 1] + 1;   // a tile for round r - 1 ...
      const long long hi = sk_tiles - (rounds - r);               // ... and one for each later round
      if (b < lo) b = lo;
      if (b > hi) b = hi;
      p->round_plan.tile_begin[r] = static_cast<int>(r == rounds ? sk_tiles : b);
    }
    for (int r = rounds + 1; r <= kMaxRounds; ++r) p->round_plan.tile_begin[r] = sk_tiles;
  }
  if (sk_tiles && p->sk_slots < p->grid) {
    cudaFree(p->sk_ws);
    cudaFree(p->sk_flags);
    p->sk_ws = nullptr;
    p->sk_flags = nullptr;
    p->sk_slots = 0;
    const size_t slot_bytes =
        sizeof(float) * 128 * static_cast<size_t>(p->layout == 2 ? kv->block_m : kv->block_n);
    // four slots per CTA (the plain schedule alternates between two of them; the cooperative
    // completion of shared tiles publishes up to two partials per round, two rounds alive),
    // a flag and a reader count per slot
    const int slots = p->max_workers * kv->cta_group * 4;
    cudaError_t e = cudaMalloc(&p->sk_ws, slot_bytes * slots);
    if (e == cudaSuccess) e = cudaMalloc(&p->sk_flags, sizeof(uint32_t) * slots * 2);
    if (e == cudaSuccess) e = cudaMemset(p->sk_flags, 0, sizeof(uint32_t) * slots * 2);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return ROLLER_ERR_NOMEM;
    }
    p->sk_slots = slots;
  }
  return ROLLER_OK;
}
