// Status strings and the small runtime surface (memory, streams, events, graphs) of the C ABI.
#include "common.cuh"
#include <string.h>
#include <stdio.h>

static thread_local char g_cuda_err[256] = "";

void b200q_set_cuda_error(cudaError_t e) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  cudaGetLastError();   // clear the sticky-free error state so later calls report their own status
}

int b200q_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { b200q_set_cuda_error(e); return -1; }
  if (dev < 0 || dev >= B200Q_MAX_DEVICES) { b200q_set_cuda_error(cudaErrorInvalidDevice); return -1; }
  return dev;
}

int b200q_sm_count() {
  static std::atomic<int> n_sm[B200Q_MAX_DEVICES];
  const int dev = b200q_current_device();
  if (dev < 0) return 0;
  int n = n_sm[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    n_sm[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

extern "C" const char* b200q_last_cuda_error(void) { return g_cuda_err; }
extern "C" int b200q_version(void) { return 1; }

extern "C" const char* b200q_strerror(int code) {
  switch (code) {
    case B200Q_OK: return "ok";
    case B200Q_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unknown enum)";
    case B200Q_ERR_BAD_SHAPE: return "shape not supported (not a multiple of the quant block, or over a kernel limit)";
    case B200Q_ERR_MISALIGNED: return "pointer not aligned as the kernel requires";
    case B200Q_ERR_UNSUPPORTED: return "quant type / dtype / option combination not supported";
    case B200Q_ERR_CUDA: return "CUDA call failed (see b200q_last_cuda_error)";
    case B200Q_ERR_TOO_LARGE: return "request exceeds a fixed capacity of the library";
    default: return "unknown b200q status";
  }
}

extern "C" int b200q_device_count(int* count) { if (!count) return B200Q_ERR_BAD_ARG; B200Q_CHECK_CUDA(cudaGetDeviceCount(count)); return B200Q_OK; }
extern "C" int b200q_set_device(int device) { B200Q_CHECK_CUDA(cudaSetDevice(device)); return B200Q_OK; }
extern "C" int b200q_device_props(int device, int* sm_count, int* cc_major, int* cc_minor, size_t* total_mem) {
  cudaDeviceProp p;
  B200Q_CHECK_CUDA(cudaGetDeviceProperties(&p, device));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  if (total_mem) *total_mem = p.totalGlobalMem;
  return B200Q_OK;
}
extern "C" int b200q_malloc(void** ptr, size_t bytes) { if (!ptr) return B200Q_ERR_BAD_ARG; B200Q_CHECK_CUDA(cudaMalloc(ptr, bytes ? bytes : 1)); return B200Q_OK; }
extern "C" int b200q_free(void* ptr) { B200Q_CHECK_CUDA(cudaFree(ptr)); return B200Q_OK; }
extern "C" int b200q_host_alloc(void** ptr, size_t bytes) { if (!ptr) return B200Q_ERR_BAD_ARG; B200Q_CHECK_CUDA(cudaMallocHost(ptr, bytes ? bytes : 1)); return B200Q_OK; }
extern "C" int b200q_host_free(void* ptr) { B200Q_CHECK_CUDA(cudaFreeHost(ptr)); return B200Q_OK; }

static int copy(void* dst, const void* src, size_t bytes, cudaMemcpyKind kind, void* stream) {
  if (bytes == 0) return B200Q_OK;
  if (!dst || !src) return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaMemcpyAsync(dst, src, bytes, kind, (cudaStream_t)stream));
  return B200Q_OK;
}
extern "C" int b200q_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream) { return copy(dst, src, bytes, cudaMemcpyHostToDevice, stream); }
extern "C" int b200q_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream) { return copy(dst, src, bytes, cudaMemcpyDeviceToHost, stream); }
extern "C" int b200q_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream) { return copy(dst, src, bytes, cudaMemcpyDeviceToDevice, stream); }
extern "C" int b200q_memset(void* dst, int value, size_t bytes, void* stream) {
  if (bytes == 0) return B200Q_OK;
  if (!dst) return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
  return B200Q_OK;
}
extern "C" int b200q_stream_create(void** stream) {
  if (!stream) return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaStreamCreateWithFlags((cudaStream_t*)stream, cudaStreamNonBlocking));
  return B200Q_OK;
}
extern "C" int b200q_stream_destroy(void* stream) { B200Q_CHECK_CUDA(cudaStreamDestroy((cudaStream_t)stream)); return B200Q_OK; }
extern "C" int b200q_stream_synchronize(void* stream) { B200Q_CHECK_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); return B200Q_OK; }
extern "C" int b200q_device_synchronize(void) { B200Q_CHECK_CUDA(cudaDeviceSynchronize()); return B200Q_OK; }
extern "C" int b200q_event_create(void** event) { if (!event) return B200Q_ERR_BAD_ARG; B200Q_CHECK_CUDA(cudaEventCreate((cudaEvent_t*)event)); return B200Q_OK; }
extern "C" int b200q_event_destroy(void* event) { B200Q_CHECK_CUDA(cudaEventDestroy((cudaEvent_t)event)); return B200Q_OK; }
extern "C" int b200q_event_record(void* event, void* stream) { B200Q_CHECK_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); return B200Q_OK; }
extern "C" int b200q_event_synchronize(void* event) { B200Q_CHECK_CUDA(cudaEventSynchronize((cudaEvent_t)event)); return B200Q_OK; }
extern "C" int b200q_event_elapsed_ms(void* start, void* stop, float* ms) {
  if (!ms) return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return B200Q_OK;
}
extern "C" int b200q_graph_begin(void* stream) {
  if (!stream) return B200Q_ERR_BAD_ARG;   // the legacy default stream cannot be captured
  B200Q_CHECK_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
  return B200Q_OK;
}
extern "C" int b200q_graph_end(void* stream, void** graph_exec) {
  if (!stream || !graph_exec) return B200Q_ERR_BAD_ARG;
  cudaGraph_t graph = nullptr;
  B200Q_CHECK_CUDA(cudaStreamEndCapture((cudaStream_t)stream, &graph));
  cudaError_t e = cudaGraphInstantiate((cudaGraphExec_t*)graph_exec, graph, 0);
  cudaGraphDestroy(graph);
  B200Q_CHECK_CUDA(e);
  return B200Q_OK;
}
extern "C" int b200q_graph_launch(void* graph_exec, void* stream) {
  if (!graph_exec) return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream));
  return B200Q_OK;
}
extern "C" int b200q_graph_destroy(void* graph_exec) { B200Q_CHECK_CUDA(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec)); return B200Q_OK; }

// ---- memory shared between the processes of one node (one process per GPU) ----
extern "C" int b200q_ipc_export(void* device_ptr, void* handle64_out) {
  if (!device_ptr || !handle64_out) return B200Q_ERR_BAD_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  cudaIpcMemHandle_t h;
  B200Q_CHECK_CUDA(cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle64_out, &h, sizeof(h));
  return B200Q_OK;
}
extern "C" int b200q_ipc_open(const void* handle64, void** device_ptr) {
  if (!handle64 || !device_ptr) return B200Q_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  B200Q_CHECK_CUDA(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return B200Q_OK;
}
extern "C" int b200q_ipc_close(void* device_ptr) {
  if (!device_ptr) return B200Q_ERR_BAD_ARG;
  B200Q_CHECK_CUDA(cudaIpcCloseMemHandle(device_ptr));
  return B200Q_OK;
}
