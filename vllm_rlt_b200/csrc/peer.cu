// Peer-memory plumbing: peer access inside one process, CUDA IPC across the
// one-process-per-GPU stage workers. It stands where the reference registers
// its pools with a NIXL agent and ships the agent metadata in the handshake
// (vllm_rlt/pd/transport.py:131-154, :162-180).

#include <cstring>

#include "common.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == RLT_IPC_HANDLE_BYTES, "IPC handle size");

extern "C" {

int rlt_peer_can_access(int device, int peer) {
  if (device < 0 || peer < 0) return RLT_E_INVALID;
  if (device == peer) return 1;
  int ok = 0;
  RLT_CUDA_TRY(cudaDeviceCanAccessPeer(&ok, device, peer));
  return ok;
}

int rlt_peer_enable(int device, int peer) {
  if (device < 0 || peer < 0) return RLT_E_INVALID;
  if (device == peer) return RLT_OK;
  int previous = 0;
  RLT_CUDA_TRY(cudaGetDevice(&previous));
  RLT_CUDA_TRY(cudaSetDevice(device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();  // clear the sticky-free error
    e = cudaSuccess;
  }
  const cudaError_t back = cudaSetDevice(previous);
  if (e != cudaSuccess) return rlt::cuda_fail(e);
  RLT_CUDA_TRY(back);
  return RLT_OK;
}

int rlt_ipc_export(const void* ptr, uint8_t handle[RLT_IPC_HANDLE_BYTES], int64_t* offset) {
  if (ptr == nullptr || handle == nullptr || offset == nullptr) return RLT_E_INVALID;
  unsigned long long base = 0;  // CUdeviceptr
  size_t size = 0;
  // The handle names the whole allocation; report where ptr sits inside it.
  cudaPointerAttributes attr;
  RLT_CUDA_TRY(cudaPointerGetAttributes(&attr, ptr));
  if (attr.type != cudaMemoryTypeDevice) return RLT_E_INVALID;
  cudaIpcMemHandle_t h;
  RLT_CUDA_TRY(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  void* range_base = nullptr;
  {
    // cudaMemGetAddressRange is not in the runtime API; the driver entry point is reached
    // through the runtime's own symbol table so that no -lcuda link is needed.
    typedef int (*GetRange)(unsigned long long*, size_t*, unsigned long long);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    RLT_CUDA_TRY(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q));
    if (fn == nullptr || q != cudaDriverEntryPointSuccess) return RLT_E_CUDA;
    if (reinterpret_cast<GetRange>(fn)(&base, &size, reinterpret_cast<unsigned long long>(ptr)) != 0) return RLT_E_CUDA;
    range_base = reinterpret_cast<void*>(base);
  }
  std::memcpy(handle, &h, RLT_IPC_HANDLE_BYTES);
  *offset = static_cast<const char*>(ptr) - static_cast<const char*>(range_base);
  return RLT_OK;
}

int rlt_ipc_open(const uint8_t handle[RLT_IPC_HANDLE_BYTES], void** base) {
  if (handle == nullptr || base == nullptr) return RLT_E_INVALID;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, RLT_IPC_HANDLE_BYTES);
  RLT_CUDA_TRY(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess));
  return RLT_OK;
}

int rlt_ipc_close(void* base) {
  if (base == nullptr) return RLT_E_INVALID;
  RLT_CUDA_TRY(cudaIpcCloseMemHandle(base));
  return RLT_OK;
}

int rlt_host_register(void* host, size_t bytes, void** device_ptr) {
  if (host == nullptr || bytes == 0 || device_ptr == nullptr) return RLT_E_INVALID;
  cudaError_t reg = cudaHostRegister(host, bytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
  if (reg == cudaErrorHostMemoryAlreadyRegistered) {
    // A mapping that was unmapped without being unregistered leaves its registration behind, and a new mapping
    // may land on the same addresses: drop the stale registration and register what is there now.
    (void)cudaGetLastError();
    (void)cudaHostUnregister(host);
    (void)cudaGetLastError();
    reg = cudaHostRegister(host, bytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
  }
  RLT_CUDA_TRY(reg);
  const cudaError_t e = cudaHostGetDevicePointer(device_ptr, host, 0);
  if (e != cudaSuccess) {
    (void)cudaHostUnregister(host);
    return rlt::cuda_fail(e);
  }
  return RLT_OK;
}

int rlt_host_unregister(void* host) {
  if (host == nullptr) return RLT_E_INVALID;
  RLT_CUDA_TRY(cudaHostUnregister(host));
  return RLT_OK;
}

}  // extern "C"
