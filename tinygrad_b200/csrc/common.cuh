// Shared declarations for the sm_100a kernels and their C-ABI launchers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <atomic>
#include "../../include/b200q.h"

#define B200Q_CHECK_CUDA(expr)                                   \
  do {                                                           \
    cudaError_t _e = (expr);                                     \
    if (_e != cudaSuccess) { b200q_set_cuda_error(_e); return B200Q_ERR_CUDA; } \
  } while (0)

void b200q_set_cuda_error(cudaError_t e);

// ---- per-device launcher state ---------------------------------------------------------
// One host process may drive several GPUs (tinygrad does: one process, one context per device,
// tinygrad/runtime/ops_cuda.py:97-134), and cudaFuncSetAttribute / the SM count belong to the device that is current.
// Launchers therefore keep what they cache in tables indexed by the current device.  Setting an attribute twice is
// harmless, so a relaxed atomic flag per device is all the thread safety the tables need.
constexpr int B200Q_MAX_DEVICES = 64;
struct PerDeviceFlag {
  std::atomic<int> v[B200Q_MAX_DEVICES];
  bool test(int dev) const { return v[dev].load(std::memory_order_acquire) != 0; }
  void set(int dev) { v[dev].store(1, std::memory_order_release); }
};
// reads and clears the status word of the decode-step kernels (decode.cu); folded into b200q_status_read_clear
int b200q_decode_status_take(int* status);
int b200q_decode_step_status_take(int* status);   // the same for the whole-step kernel (decode_step.cu)
int b200q_peer_status_take(int* status);          // the same for the peer-memory collectives (peer.cu)
int b200q_ep_status_take(int* status);            // the same for the expert-parallel exchange (ep.cu)
// current device index, or -1 (with the CUDA error recorded) if it cannot be had or is past the tables
int b200q_current_device();
// SM count of the current device (cached per device); 0 on error
int b200q_sm_count();

// ---- packed weight layout (see include/b200q.h for the byte-level description)
constexpr int TILE_ROWS = 16;       // output rows per tile (one mma.m16n8k16 A operand)
constexpr int GROUP_ELEMS = 128;    // K elements per tile: 4 quant blocks of 32 (Q4_0/Q8_0), half a super-block (Q6_K)

__host__ __device__ constexpr int tile_bytes(int qtype) {
  return qtype == B200Q_Q4_0 ? 1152 : qtype == B200Q_Q8_0 ? 2176 : qtype == B200Q_Q6_K ? 1696 : 0;
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch (PDL).  Every kernel calls pdl_wait() before it
// touches memory another kernel wrote, so a chain of launches stays ordered.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch with the programmatic-stream-serialization attribute when `pdl` is set.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                                   Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- mailboxes in peer memory ---------------------------------------------------------------------------------------
// A mailbox word is 32 bits: the fp32 value, or MAILBOX_EMPTY.  One aligned 32-bit store / load is atomic, so a word is either
// empty or complete: the reader polls the data itself, no flag and no fence, and puts MAILBOX_EMPTY back when it has read it.
// The all-ones pattern is a NaN no arithmetic produces (results that are NaN travel as the canonical quiet NaN).
constexpr uint32_t MAILBOX_EMPTY = 0xFFFFFFFFu;
__device__ __forceinline__ uint32_t mailbox_bits(float v) { const uint32_t b = __float_as_uint(v); return b == MAILBOX_EMPTY ? 0x7FC00000u : b; }
__device__ __forceinline__ void mailbox_store(uint32_t* p, uint32_t bits) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(bits) : "memory"); }
__device__ __forceinline__ uint32_t mailbox_load(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {   // weights are read once: do not keep them in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
