// Symmetric peer memory for the tensor-parallel ranks of one node: every rank allocates a region, exports a CUDA IPC
// handle and maps the regions of all peers, so kernels can store into and load from peer memory over NVLink.
// Reference counterpart: ak_tp_region_alloc / ak_tp_region_open / ak_tp_can_peer (kernels/src/tp_ar.cu:236-288) with
// the rendezvous of crates/agens-cli/src/tp.rs:94-175; here the handles travel through torch.distributed.
#include "../kernels/sm100/common.cuh"

using namespace b2;

B2_API int b2_ipc_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64 || bytes == 0) return B2_ERR_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return B2_ERR_LAUNCH;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return B2_ERR_LAUNCH; }
  static_assert(sizeof(h) == 64, "CUDA IPC handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return B2_OK;
}

B2_API int b2_ipc_open(const unsigned char* handle64, void** ptr) {
  if (!ptr || !handle64) return B2_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH;
}

B2_API int b2_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH; }
B2_API int b2_ipc_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? B2_OK : B2_ERR_LAUNCH; }

B2_API int b2_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}
