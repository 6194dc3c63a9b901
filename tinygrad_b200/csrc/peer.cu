// Collectives over peer memory: the consumer side of the mailboxes that sharded linears fill (gemv.cu, `peer` epilogue).
//
// Replaces the reference's schedule-time expansion of a sharded reduce into device-to-device copies and add kernels
// (tinygrad/schedule/allreduce.py:6-58).  At batch 1 a tensor-parallel decode step holds ~160 reductions of one 16-32 KB
// vector: latency is everything.  Here the producing GEMV stores each finished value straight into a mailbox on every rank
// (plain 32-bit stores over NVLink, no staging, no library call), and this kernel -- one launch, a few CTAs, under programmatic
// dependent launch -- polls its local mailbox until every rank's word is there, adds them in rank order (so all ranks compute
// bit-identical sums) and puts the empty pattern back for the next step.  There is no flag, no fence and no barrier: a word is
// either the empty pattern or a complete value.  Every poll is bounded; on expiry the status word is raised and the word
// counts as zero.
#include "common.cuh"

namespace {

constexpr int MR_THREADS = 256;
constexpr int MR_DEFAULT_SPIN = 1 << 22;

__device__ int g_peer_status = 0;

__global__ void __launch_bounds__(MR_THREADS) mailbox_reduce_kernel(uint32_t* __restrict__ mailbox, int n_slots, int n, const float* __restrict__ residual,
                                                                    float* __restrict__ out, int spin_limit) {
  pdl_launch_dependents();
  pdl_wait();                      // the residual (and, for this rank's own slot, the producer) come from earlier launches
  const int i = blockIdx.x * MR_THREADS + threadIdx.x;
  if (i >= n) return;
  float acc = residual ? residual[i] : 0.f;
  // all slots' loads are issued before any is examined: one round trip when the words are there already
  uint32_t w[B200Q_MAX_PEERS];
#pragma unroll
  for (int r = 0; r < B200Q_MAX_PEERS; r++) if (r < n_slots) w[r] = mailbox_load(mailbox + (size_t)r * n + i);
#pragma unroll
  for (int r = 0; r < B200Q_MAX_PEERS; r++) {
    if (r >= n_slots) break;
    uint32_t v = w[r];
    uint32_t* word = mailbox + (size_t)r * n + i;
    for (int k = 0; v == MAILBOX_EMPTY && k < spin_limit; k++) {
      if (k > 64) __nanosleep(100);
      v = mailbox_load(word);
    }
    if (v == MAILBOX_EMPTY) { atomicExch(&g_peer_status, 1); v = 0u; }
    acc += __uint_as_float(v);
    mailbox_store(word, MAILBOX_EMPTY);      // ready for the next step (the next writer is at least one whole collective away)
  }
  out[i] = acc;
}

}  // namespace

int b200q_peer_status_take(int* status) {
  int zero = 0;
  B200Q_CHECK_CUDA(cudaMemcpyFromSymbol(status, g_peer_status, sizeof(int)));
  B200Q_CHECK_CUDA(cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int)));
  return B200Q_OK;
}

extern "C" int b200q_mailbox_reduce(void* mailbox, int n_slots, int n, const float* residual, float* out, int spin_limit, int flags, void* stream) {
  if (!mailbox || !out || n <= 0 || n_slots <= 0 || n_slots > B200Q_MAX_PEERS || spin_limit < 0) return B200Q_ERR_BAD_ARG;
  if ((uintptr_t)mailbox & 3) return B200Q_ERR_MISALIGNED;
  B200Q_CHECK_CUDA(launch_k(mailbox_reduce_kernel, dim3(ceil_div(n, MR_THREADS)), dim3(MR_THREADS), 0, (cudaStream_t)stream, (flags & B200Q_FLAG_PDL) != 0,
                            (uint32_t*)mailbox, n_slots, n, residual, out, spin_limit ? spin_limit : MR_DEFAULT_SPIN));
  return B200Q_OK;
}
