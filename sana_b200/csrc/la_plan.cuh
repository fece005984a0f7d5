// Host-side launch planning shared by the linear-attention kernels.
#pragma once
#include "common.cuh"

namespace sana {

// Host-side split of the token axis into chunks of Lc tokens (a multiple of 64).  `units` CTAs
// exist per chunk (samples x head groups) and `slots` CTAs are resident at once; a CTA's time is
// its Lc tokens plus a fixed cost of `overhead` token-equivalents (state load, or partial-state
// write + re-read).  Picks the chunk count that minimises waves x (Lc + overhead), i.e. avoids
// a mostly empty last wave.
inline void la_chunking(int64_t units, int64_t N, int64_t slots, int64_t overhead, int* Lc, int* nchunks) {
  const int64_t max_chunks = ceil_div(N, 64) < 4096 ? ceil_div(N, 64) : 4096;
  int64_t best_cost = -1, best_lc = 64;
  for (int64_t nch = 1; nch <= max_chunks; ++nch) {
    const int64_t lc = ceil_div(ceil_div(N, nch), 64) * 64;
    const int64_t real = ceil_div(N, lc);
    const int64_t cost = ceil_div(units * real, slots) * (lc + overhead);
    if (best_cost < 0 || cost < best_cost) best_cost = cost, best_lc = lc;
  }
  *Lc = (int)best_lc;
  *nchunks = (int)ceil_div(N, best_lc);
}

template <typename Kernel>
inline int64_t resident_ctas(Kernel kernel, int threads, size_t dynamic_smem = 0) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, dynamic_smem) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    per_sm = 1;
  }
  return (int64_t)per_sm * sm_count();
}

// The same for a kernel that allocates `tmem_cols` columns of tensor memory: the runtime's occupancy
// query answers 1 for such kernels whatever they allocate, so the limits are applied here - 64 K
// registers (allocated per warp in units of 8 per thread), 228 KiB of shared memory of which
// every resident CTA also takes 1 KiB for the system, 2048 threads, 512 tensor-memory columns.
template <typename Kernel>
inline int64_t resident_ctas_tmem(Kernel kernel, int threads, size_t dynamic_smem, int tmem_cols) {
  cudaFuncAttributes attr;
  if (cudaFuncGetAttributes(&attr, kernel) != cudaSuccess) {
    cudaGetLastError();
    return sm_count();
  }
  const int64_t regs = ((int64_t)(attr.numRegs > 0 ? attr.numRegs : 32) + 7) / 8 * 8;
  int64_t per_sm = 65536 / (regs * threads);
  const int64_t by_smem = (228 * 1024) / (int64_t)(dynamic_smem + attr.sharedSizeBytes + 1024);
  if (by_smem < per_sm) per_sm = by_smem;
  if (2048 / threads < per_sm) per_sm = 2048 / threads;
  if (512 / tmem_cols < per_sm) per_sm = 512 / tmem_cols;
  if (per_sm < 1) per_sm = 1;
  return per_sm * sm_count();
}

// Chunk reduction fused with the all-reduce over peer memory (la_core.cu), shared by the linear-attention state
// kernels: sums the `nchunks` partial states of this rank in chunk order, publishes the sum in this rank's
// exchange buffer and adds the peers' sums in rank order.  `peer_buffers[r]` = rank r's exchange buffer
// (SP_HEADER_BYTES + 2 * total * 4 bytes, zeroed before the first step) as mapped in this process.
constexpr int SP_MAX_WORLD = 16;
constexpr int64_t SP_HEADER_BYTES = 1024;
int launch_state_reduce_exchange(const float* partial, float* state, int nchunks, int64_t per_batch, int64_t total,
                                 void* const* peer_buffers, int rank, int world, uint32_t step, cudaStream_t st);

}  // namespace sana
