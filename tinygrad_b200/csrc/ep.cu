// Expert-parallel exchange for the MXFP8 mixture-of-experts layer, over peer memory (NVLink), planned on the device.
//
// The reference's grouped path routes and regroups tokens on ONE device (`route` / `dispatch` / `combine`,
// extra/gemm/moe_routing.py:109-131); it has no expert-parallel exchange.  Here experts are split contiguously over the ranks and
// tokens over the ranks at the input, and `dispatch` / `combine` cross the ranks without a communication library and without the
// host reading anything:
//   1. every rank routes its own tokens (b200q_moe_route_pad, compact expert-sorted order) and PUBLISHES its per-expert row counts
//      into a mailbox on every rank (self-validating 32-bit words, common.cuh);
//   2. a one-CTA PLAN kernel waits for all ranks' counts and derives, on every rank alike, where each (source rank, expert) run of
//      rows starts inside the owning rank's grouped buffer (groups padded to 256 rows, sources in rank order: the placement the
//      single-device `route` would give the concatenated tokens) and the local group offsets the expert GEMMs take;
//   3. DISPATCH quantises each token row once (E4M3 + E8M0) and stores it straight into the owning ranks' GEMM operand buffers
//      (16-byte stores over NVLink), then raises a "rows landed" flag on every rank; a WAIT kernel on the receiver consumes the flags;
//   4. the grouped expert GEMMs run on the local groups (mxfp8_gemm.cu); a SIGNAL kernel tells every rank the results stand;
//   5. COMBINE on the token-owning rank waits for those flags and PULLS its k result rows per token from the owning ranks' buffers
//      (16-byte loads over NVLink), weights and adds them in slot order.
// Every row's arithmetic is the single-device path's, so the result is bit-identical to it.  All waits are bounded.
#include "common.cuh"
#include "mxq.cuh"
#include <cuda_bf16.h>

namespace {

constexpr int EP_SPIN = 1 << 22;
constexpr int EP_BLOCK_ROW = 256;      // extra/gemm/moe_routing.py:4

__device__ int g_ep_status = 0;

struct EpPtrs {                        // per rank, as mapped into this process
  uint32_t* counts[B200Q_MAX_PEERS];   // mailbox words [n_ranks][n_experts]
  uint8_t* a_q[B200Q_MAX_PEERS];       // [m_max][d]
  uint8_t* a_e8[B200Q_MAX_PEERS];      // [m_max][d / 32]
  const __nv_bfloat16* y[B200Q_MAX_PEERS];   // [m_max][d]
  uint32_t* flags[B200Q_MAX_PEERS];    // [2][n_ranks]: rows landed, results ready
};

__device__ __forceinline__ uint32_t ld_sys(const uint32_t* p) { return mailbox_load(p); }
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void ep_publish_kernel(EpPtrs pp, const int32_t* __restrict__ counts, int n_ranks, int rank, int n_experts) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_experts) return;
  const uint32_t c = (uint32_t)counts[e];
  for (int d = 0; d < n_ranks; d++) mailbox_store(pp.counts[d] + (size_t)rank * n_experts + e, c);
}

// One CTA.  Thread e: total rows of expert e over all ranks, rows of lower ranks before this rank's, then the padded group starts.
__global__ void ep_plan_kernel(uint32_t* __restrict__ counts_all, int n_ranks, int rank, int n_experts, int32_t* __restrict__ send_base,
                               int32_t* __restrict__ off_local) {
  extern __shared__ int s_pad[];       // [n_experts] padded group size of every expert
  const int e_l = n_experts / n_ranks;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    int total = 0;
    for (int s = 0; s < n_ranks; s++) {
      uint32_t* w = counts_all + (size_t)s * n_experts + e;
      uint32_t v = ld_sys(w);
      for (int i = 0; v == MAILBOX_EMPTY && i < EP_SPIN; i++) { if (i > 64) __nanosleep(100); v = ld_sys(w); }
      if (v == MAILBOX_EMPTY) { atomicExch(&g_ep_status, 1); v = 0; }
      total += (int)v;
    }
    s_pad[e] = (total + EP_BLOCK_ROW - 1) / EP_BLOCK_ROW * EP_BLOCK_ROW;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int d = e / e_l, le = e - d * e_l;
    int base = 0;
    for (int j = 0; j < le; j++) base += s_pad[d * e_l + j];
    int before = 0;
    for (int s = 0; s < rank; s++) { const uint32_t v = ld_sys(counts_all + (size_t)s * n_experts + e); before += v == MAILBOX_EMPTY ? 0 : (int)v; }
    send_base[e] = base + before;
    if (d == rank) { off_local[le] = base; if (le == e_l - 1) off_local[e_l] = base + s_pad[e]; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_ranks * n_experts; i += blockDim.x) mailbox_store(counts_all + i, MAILBOX_EMPTY);      // ready for the next layer
}

// Quantise the local token rows (bf16) and store each into the grouped operand buffer of the rank that owns its expert.
// One warp per 256 consecutive values of a row, as quantize_mxfp8_kernel; the E8M0 bytes of a warp's 8 blocks go out as one 8-byte store.
__global__ void ep_dispatch_kernel(EpPtrs pp, const __nv_bfloat16* __restrict__ x, int n_tokens, int d_model, int k, int n_experts, int n_ranks, int rank,
                                   const int32_t* __restrict__ topi, const int32_t* __restrict__ dest, const int32_t* __restrict__ off,
                                   const int32_t* __restrict__ send_base, int32_t* __restrict__ remote_row, unsigned* __restrict__ done, int m_max) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int kb = d_model >> 5, chunks = kb >> 3, e_l = n_experts / n_ranks;      // d_model % 256 == 0
  if (warp < (int64_t)n_tokens * chunks) {
    const int64_t r = warp / chunks;
    const int chunk = (int)(warp - r * chunks), b = chunk * 8 + (lane >> 2), col = b * 32 + (lane & 3) * 8;
    float v[8];
    const uint4 u = *reinterpret_cast<const uint4*>(x + r * d_model + col);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(v[i]));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
    const uint8_t e = mx_scale_exponent(m);
    const uint2 pk = mx_quant8(v, e);
    // the 8 scale bytes of this warp's blocks, gathered into lanes 0 and 1 (4 bytes each)
    uint32_t sc = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) sc |= (uint32_t)__shfl_sync(0xffffffffu, (uint32_t)e, ((lane & 1) * 4 + j) * 4) << (8 * j);
    for (int f = 0; f < k; f++) {
      const int64_t idx = r * k + f;
      const int ex = topi[idx], dr = ex / e_l;
      const int row = send_base[ex] + (dest[idx] - off[ex]);
      if (row < 0 || row >= m_max) { atomicExch(&g_ep_status, 2); continue; }       // a plan that does not fit the buffers: skip, flag
      if (chunk == 0 && lane == 0) remote_row[idx] = row;
      *reinterpret_cast<uint2*>(pp.a_q[dr] + (size_t)row * d_model + col) = pk;
      if (lane < 2) *reinterpret_cast<uint32_t*>(pp.a_e8[dr] + (size_t)row * kb + chunk * 8 + lane * 4) = sc;
    }
  }
  // "rows landed": the last CTA to get here, after everybody's stores are visible system-wide, raises this rank's flag on every rank
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(done, 1u);
    s_last = prev == gridDim.x - 1;
    if (s_last) *done = 0;
  }
  __syncthreads();
  if (s_last && threadIdx.x < n_ranks) { __threadfence_system(); st_release_sys(pp.flags[threadIdx.x] + rank, 1u); }
}

// Consume the flags of kind `which` (0 rows landed, 1 results ready) from every rank; the launches behind it in the stream may then read.
__global__ void ep_wait_kernel(uint32_t* __restrict__ flags, int n_ranks, int which, int spin) {
  const int s = threadIdx.x;
  if (s >= n_ranks) return;
  uint32_t* w = flags + (size_t)which * n_ranks + s;
  uint32_t v = ld_acquire_sys(w);
  for (int i = 0; v == 0 && i < spin; i++) { if (i > 64) __nanosleep(100); v = ld_acquire_sys(w); }
  if (v == 0) atomicExch(&g_ep_status, 1);
  *w = 0;                                   // the next raise of this flag is at least one whole exchange away
  __threadfence_system();
}

__global__ void ep_signal_kernel(EpPtrs pp, int n_ranks, int rank) {
  if (threadIdx.x < n_ranks) { __threadfence_system(); st_release_sys(pp.flags[threadIdx.x] + n_ranks + rank, 1u); }
}

// out[t] = sum_j weights[t, j] * y_{owner(j)}[remote_row[t, j]], fp32 sum in slot order, bf16 in / out (`combine`, moe_routing.py:128-131)
__global__ void ep_combine_kernel(EpPtrs pp, const int32_t* __restrict__ topi, const int32_t* __restrict__ remote_row, const float* __restrict__ weights,
                                  int n_tokens, int k, int d_model, int e_l, __nv_bfloat16* __restrict__ out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < d_model; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; j++) {
      const size_t idx = (size_t)t * k + j;
      const float w = weights[idx];
      const uint4 u = *reinterpret_cast<const uint4*>(pp.y[topi[idx] / e_l] + (size_t)remote_row[idx] * d_model + c);
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int i = 0; i < 4; i++) { acc[2 * i] += w * __uint_as_float(ww[i] << 16); acc[2 * i + 1] += w * __uint_as_float(ww[i] & 0xFFFF0000u); }
    }
    uint4 pk;
    __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int i = 0; i < 4; i++) hp[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)t * d_model + c) = pk;
  }
}

int fill_ptrs(const b200q_ep_args* a, EpPtrs& pp) {
  for (int d = 0; d < a->n_ranks; d++) {
    if (!a->counts_all[d] || !a->a_q[d] || !a->a_e8[d] || !a->y[d] || !a->flags[d]) return B200Q_ERR_BAD_ARG;
    pp.counts[d] = (uint32_t*)a->counts_all[d]; pp.a_q[d] = (uint8_t*)a->a_q[d]; pp.a_e8[d] = (uint8_t*)a->a_e8[d];
    pp.y[d] = (const __nv_bfloat16*)a->y[d]; pp.flags[d] = (uint32_t*)a->flags[d];
  }
  return B200Q_OK;
}

int check_args(const b200q_ep_args* a) {
  if (!a || !a->counts_all || !a->a_q || !a->a_e8 || !a->y || !a->flags) return B200Q_ERR_BAD_ARG;
  if (a->n_ranks <= 0 || a->n_ranks > B200Q_MAX_PEERS || a->rank < 0 || a->rank >= a->n_ranks) return B200Q_ERR_BAD_ARG;
  if (a->n_experts <= 0 || a->n_experts % a->n_ranks || a->n_experts > 1024 || a->k <= 0 || a->n_tokens <= 0 || a->m_max <= 0) return B200Q_ERR_BAD_ARG;
  if (a->d_model <= 0 || a->d_model % 256) return B200Q_ERR_BAD_SHAPE;
  return B200Q_OK;
}

}  // namespace

int b200q_ep_status_take(int* status) {
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_ep_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_ep_status, &zero, sizeof(int)));
  return B200Q_OK;
}

extern "C" int b200q_ep_publish_counts(const b200q_ep_args* a, void* stream) {
  int rc = check_args(a); if (rc) return rc;
  if (!a->counts) return B200Q_ERR_BAD_ARG;
  EpPtrs pp; rc = fill_ptrs(a, pp); if (rc) return rc;
  ep_publish_kernel<<<ceil_div(a->n_experts, 256), 256, 0, (cudaStream_t)stream>>>(pp, a->counts, a->n_ranks, a->rank, a->n_experts);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_ep_plan(const b200q_ep_args* a, void* stream) {
  int rc = check_args(a); if (rc) return rc;
  if (!a->send_base || !a->off_local) return B200Q_ERR_BAD_ARG;
  ep_plan_kernel<<<1, 256, a->n_experts * sizeof(int), (cudaStream_t)stream>>>((uint32_t*)a->counts_all[a->rank], a->n_ranks, a->rank, a->n_experts, a->send_base,
                                                                               a->off_local);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_ep_dispatch(const b200q_ep_args* a, const void* x_bf16, void* stream) {
  int rc = check_args(a); if (rc) return rc;
  if (!x_bf16 || !a->topi || !a->dest || !a->off || !a->send_base || !a->remote_row || !a->scratch) return B200Q_ERR_BAD_ARG;
  if ((uintptr_t)x_bf16 & 15) return B200Q_ERR_MISALIGNED;
  EpPtrs pp; rc = fill_ptrs(a, pp); if (rc) return rc;
  const int64_t warps = (int64_t)a->n_tokens * (a->d_model / 256);
  ep_dispatch_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, (cudaStream_t)stream>>>(pp, (const __nv_bfloat16*)x_bf16, a->n_tokens, a->d_model, a->k, a->n_experts,
                                                                                  a->n_ranks, a->rank, a->topi, a->dest, a->off, a->send_base, a->remote_row,
                                                                                  (unsigned*)a->scratch, a->m_max);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_ep_wait(const b200q_ep_args* a, int which, int spin_limit, void* stream) {
  int rc = check_args(a); if (rc) return rc;
  if ((which != 0 && which != 1) || spin_limit < 0) return B200Q_ERR_BAD_ARG;
  ep_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint32_t*)a->flags[a->rank], a->n_ranks, which, spin_limit ? spin_limit : EP_SPIN);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_ep_signal_results(const b200q_ep_args* a, void* stream) {
  int rc = check_args(a); if (rc) return rc;
  EpPtrs pp; rc = fill_ptrs(a, pp); if (rc) return rc;
  ep_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pp, a->n_ranks, a->rank);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}

extern "C" int b200q_ep_combine(const b200q_ep_args* a, const float* weights, void* out_bf16, void* stream) {
  int rc = check_args(a); if (rc) return rc;
  if (!weights || !out_bf16 || !a->topi || !a->remote_row) return B200Q_ERR_BAD_ARG;
  EpPtrs pp; rc = fill_ptrs(a, pp); if (rc) return rc;
  ep_combine_kernel<<<a->n_tokens, 256, 0, (cudaStream_t)stream>>>(pp, a->topi, a->remote_row, weights, a->n_tokens, a->k, a->d_model, a->n_experts / a->n_ranks,
                                                                  (__nv_bfloat16*)out_bf16);
  B200Q_CHECK_CUDA(cudaGetLastError());
  return B200Q_OK;
}
