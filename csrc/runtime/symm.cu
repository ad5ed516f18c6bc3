// Symmetric-memory substrate: device allocations that every rank of a node can address
// (CUDA IPC handles exchanged by the Python layer over the process group) and the cross-rank
// barrier kernel. Plays the role of the reference's src/ths_op/flux_shm.cc
// (cudaipc_create_tensor_list) and src/cuda/cudaipc_barrier_all.cu, without the CAS-reset
// protocol: flags carry the call number and only ever grow, and every wait is bounded.
#include "../include/fluxb.h"
#include "../sm100/ptx.cuh"
#include "host_common.h"

#include <atomic>

namespace fluxb {
extern std::atomic<uint64_t> g_launches;

__global__ void barrier_all_kernel(uint32_t* f0,
                                   uint32_t* f1, uint32_t* f2, uint32_t* f3, uint32_t* f4,
                                   uint32_t* f5, uint32_t* f6, uint32_t* f7, int rank, int world,
                                   uint32_t epoch, uint64_t timeout_ns, Status* status) {
  __shared__ uint32_t abort_word;
  uint32_t* flags[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
  if (threadIdx.x == 0) abort_word = 0;
  __syncwarp();
  const int lane = threadIdx.x;
  WaitCtx wc{status, &abort_word, timeout_ns};
  // everything this rank wrote before the barrier must be visible to whoever sees the flag
  __threadfence_system();
  if (lane < world) {
    ptx::st_release_sys(flags[lane] + rank, epoch);
    flag_wait_ge(wc, flags[rank] + lane, epoch, kSiteBarrierAll);
  }
  __syncwarp();
  __threadfence_system();
}

__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns,
                                 Status* status) {
  __shared__ uint32_t abort_word;
  abort_word = 0;
  WaitCtx wc{status, &abort_word, timeout_ns};
  flag_wait_ge(wc, flag, expected, kSiteTest);
}

}  // namespace fluxb

using namespace fluxb;

extern "C" int fluxb_symm_alloc(uint64_t bytes, void** ptr, void* handle) {
  FLUXB_REQUIRE(ptr && handle && bytes > 0, "symm_alloc arguments");
  void* p = nullptr;
  FLUXB_CUDA_OK(cudaMalloc(&p, bytes));
  FLUXB_CUDA_OK(cudaMemset(p, 0, bytes));
  FLUXB_CUDA_OK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(kErrCuda, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return kOk;
}

extern "C" int fluxb_symm_open(const void* handle, void** ptr) {
  FLUXB_REQUIRE(ptr && handle, "symm_open arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  FLUXB_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return kOk;
}

extern "C" int fluxb_symm_close(void* ptr) {
  FLUXB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return kOk;
}

extern "C" int fluxb_symm_free(void* ptr) {
  FLUXB_CUDA_OK(cudaFree(ptr));
  return kOk;
}

extern "C" int fluxb_can_access_peer(int dev, int peer, int* out) {
  FLUXB_REQUIRE(out != nullptr, "null out");
  FLUXB_CUDA_OK(cudaDeviceCanAccessPeer(out, dev, peer));
  return kOk;
}

extern "C" int fluxb_barrier_all(uint32_t* const* flags, int rank, int world, uint32_t epoch,
                                 uint64_t timeout_ns, fluxb_status_t* status, void* stream) {
  FLUXB_REQUIRE(flags && world >= 1 && world <= FLUXB_MAX_RANKS && rank >= 0 && rank < world,
                "barrier arguments");
  uint32_t* f[8] = {nullptr};
  for (int i = 0; i < world; ++i) {
    FLUXB_REQUIRE(flags[i] != nullptr, "barrier flag pointer");
    f[i] = flags[i];
  }
  barrier_all_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], rank, world, epoch,
      timeout_ns ? timeout_ns : 2000000000ull, reinterpret_cast<Status*>(status));
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

// Wait until *flag == expected (not "at least": a larger value left over from an earlier exchange
// does not satisfy the wait). One thread, system-scope acquire loads, bounded.
__global__ void wait_flag_eq_kernel(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns, Status* status) {
  __shared__ uint32_t abort_word;
  abort_word = 0;
  WaitCtx wc{status, &abort_word, timeout_ns};
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t v = ptx::ld_acquire_sys(flag);
  uint32_t spins = 0;
  while (v != expected) {
    if ((++spins & 31u) == 0u && ptx::globaltimer_ns() - t0 > timeout_ns) {
      wait_give_up(wc, kSiteTest, v, expected);
      return;
    }
    __nanosleep(40);
    v = ptx::ld_acquire_sys(flag);
  }
}

extern "C" int fluxb_wait_flag_eq(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns,
                                  fluxb_status_t* status, void* stream) {
  FLUXB_REQUIRE(flag != nullptr, "flag pointer");
  wait_flag_eq_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      flag, expected, timeout_ns ? timeout_ns : 1000000000ull, reinterpret_cast<Status*>(status));
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}

extern "C" int fluxb_wait_flag(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns,
                               fluxb_status_t* status, void* stream) {
  FLUXB_REQUIRE(flag != nullptr, "flag pointer");
  wait_flag_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      flag, expected, timeout_ns ? timeout_ns : 1000000000ull, reinterpret_cast<Status*>(status));
  FLUXB_CUDA_OK(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return kOk;
}
