// Arrival flags between the GPUs of a node: a rank tells another that its stores into that
// rank's memory are complete, and a rank waits -- bounded -- for such flags. The multi-GPU
// driver closes its fused exchange of C with them: a 4-byte store per rank over NVLink in
// place of a collective. See include/roller_b200.h for the contract.
#include "../../include/roller_b200.h"

#include "gemm_launch.h"
#include "ptx_sm100.cuh"

namespace {

using namespace rb200;

struct FlagTargets {
  uint32_t* dst[ROLLER_MAX_FLAG_TARGETS];
};

// Thread i stores `value` into target i with system-scope release semantics: everything this
// GPU wrote before (the preceding kernels of the stream have completed, and with them their
// stores into the peer's memory) is visible to whoever acquires the flag.
__global__ void flag_signal_kernel(FlagTargets t, int n, uint32_t value) {
  const int i = static_cast<int>(threadIdx.x);
  if (i < n) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(t.dst[i]), "r"(value) : "memory");
  }
}

// Thread i waits until flag i has reached `value` (flags count steps, so "reached" is a
// wrap-safe comparison), at most `limit` clock cycles; a wait that runs out records
// kDevTimeoutPeer in *status and the kernel returns all the same.
__global__ void flag_wait_kernel(const uint32_t* flags, int n, unsigned long long mask,
                                 uint32_t value, long long limit, uint32_t* status) {
  const int i = static_cast<int>(threadIdx.x);
  if (i >= n || !((mask >> i) & 1ull)) return;
  const long long t0 = clock64();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
    if (static_cast<int32_t>(v - value) >= 0) return;
    if (clock64() - t0 > limit) {
      atomicCAS(status, kDevOk, kDevTimeoutPeer);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace

extern "C" {

int roller_b200_flag_signal_async(uint32_t* const* targets, int n, uint32_t value, void* stream) {
  if (!targets || n <= 0 || n > ROLLER_MAX_FLAG_TARGETS) return ROLLER_ERR_INVALID;
  FlagTargets t = {};
  for (int i = 0; i < n; ++i) {
    if (!targets[i] || (reinterpret_cast<uintptr_t>(targets[i]) & 3)) return ROLLER_ERR_INVALID;
    t.dst[i] = targets[i];
  }
  flag_signal_kernel<<<1, ROLLER_MAX_FLAG_TARGETS, 0, static_cast<cudaStream_t>(stream)>>>(t, n, value);
  return cudaGetLastError() == cudaSuccess ? ROLLER_OK : ROLLER_ERR_CUDA;
}

int roller_b200_flag_wait_async(const uint32_t* flags, int n, unsigned long long mask,
                                uint32_t value, long long limit_cycles, uint32_t* dev_status,
                                void* stream) {
  if (!flags || !dev_status || n <= 0 || n > 64 || limit_cycles < 0) return ROLLER_ERR_INVALID;
  const long long limit = limit_cycles == 0 ? kSpinLimitCycles : limit_cycles;
  flag_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(flags, n, mask, value, limit,
                                                                   dev_status);
  return cudaGetLastError() == cudaSuccess ? ROLLER_OK : ROLLER_ERR_CUDA;
}

}  // extern "C"
