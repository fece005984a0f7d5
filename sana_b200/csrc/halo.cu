// Sequence-parallel conv halo over peer memory: every rank pushes its first / last image row of
// the depthwise conv's input into the neighbours' halo slots with plain remote stores, tells
// them with a release-store of the step number, and waits (bounded) for their rows - one
// kernel per step, no NCCL call, no multicast, no TMA.
//
// Buffer of a rank (mapped by its two neighbours; zero-filled once before the first step):
//   [0, 4)    last step whose row the UPPER neighbour (rank - 1) has delivered into `top`
//   [4, 8)    last step whose row the LOWER neighbour (rank + 1) has delivered into `bot`
//   [8, 12)   block counter   [12, 16) exit counter   [16, 20) last completed step
//   [20, 24)  soft-error word (bit 0 = the upper, bit 1 = the lower neighbour did not arrive in time)
//   [1024, 1024 + row_bytes)                  `top`: the row above this rank's first row
//   [1024 + row_bytes, 1024 + 2 * row_bytes)  `bot`: the row below its last row
// One slot per side is enough: a neighbour writes step s+1's row only after its next
// linear-attention state exchange, which cannot complete before this rank has published its
// own state of step s+1 - and it does that, in stream order, after its conv of step s has
// consumed the slot.
#include "common.cuh"

namespace sana {

constexpr int64_t HALO_HEADER_BYTES = 1024;

struct HaloArgs {
  const uint4* first_row;  // this rank's first row (goes to the upper neighbour's `bot`), or null
  const uint4* last_row;   // this rank's last row (goes to the lower neighbour's `top`), or null
  unsigned char* mine;
  unsigned char* upper;    // rank - 1's buffer, or null
  unsigned char* lower;    // rank + 1's buffer, or null
  int64_t row_vecs;        // 16-byte vectors per row
  uint32_t step;           // 0 = numbered by the kernel
  long long wait_limit_ns; // how long the waiting block waits for each neighbour
};

__device__ __forceinline__ uint32_t halo_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void halo_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ long long halo_ns() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(256) halo_exchange_kernel(const HaloArgs a) {
  uint32_t* hdr = reinterpret_cast<uint32_t*>(a.mine);
  // the step word only changes when the last block of a launch exits
  const uint32_t step = a.step ? a.step : *reinterpret_cast<volatile uint32_t*>(hdr + 4) + 1u;
  const int64_t row_bytes = a.row_vecs * 16;
  // ---- push: my first row is the upper neighbour's `bot`, my last row the lower one's `top`
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
  if (a.upper) {
    uint4* dst = reinterpret_cast<uint4*>(a.upper + HALO_HEADER_BYTES + row_bytes);
    for (int64_t i = tid; i < a.row_vecs; i += nthreads) dst[i] = a.first_row[i];
  }
  if (a.lower) {
    uint4* dst = reinterpret_cast<uint4*>(a.lower + HALO_HEADER_BYTES);
    for (int64_t i = tid; i < a.row_vecs; i += nthreads) dst[i] = a.last_row[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(hdr + 2, 1u) == gridDim.x - 1) {  // both rows are written: tell the neighbours
      hdr[2] = 0u;
      __threadfence_system();
      if (a.upper) halo_st_release(reinterpret_cast<uint32_t*>(a.upper) + 1, step);  // I am its lower neighbour
      if (a.lower) halo_st_release(reinterpret_cast<uint32_t*>(a.lower) + 0, step);  // I am its upper neighbour
      // ---- wait for the neighbours' rows (their flags arrive in my own memory)
      // each side has its own clock, and the soft-error word collects one bit per side
      for (int side = 0; side < 2; ++side) {
        if (!(side == 0 ? a.upper : a.lower)) continue;
        const long long t0 = halo_ns();
        while ((int32_t)(halo_ld_acquire(hdr + side) - step) < 0) {
          if (halo_ns() - t0 > a.wait_limit_ns) {
            atomicOr(reinterpret_cast<int*>(hdr + 5), 1 << side);
            break;
          }
        }
      }
    }
    if (atomicAdd(hdr + 3, 1u) == gridDim.x - 1) {  // the last block to leave records the step
      hdr[3] = 0u;
      *reinterpret_cast<volatile uint32_t*>(hdr + 4) = step;
    }
  }
}

}  // namespace sana

using namespace sana;

extern "C" int64_t sana_halo_exchange_buffer_bytes(int64_t row_bytes) {
  if (row_bytes <= 0) return 0;
  return HALO_HEADER_BYTES + 2 * ((row_bytes + 15) / 16 * 16);
}

extern "C" int sana_halo_exchange(const void* first_row, const void* last_row, int64_t row_bytes, void* mine,
                                  void* upper, void* lower, uint32_t step, void* stream) {
  SANA_REQUIRE(mine, "sana_halo_exchange: null buffer");
  SANA_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "sana_halo_exchange: a row must be a multiple of 16 bytes");
  SANA_REQUIRE(!upper || first_row, "sana_halo_exchange: first_row required with an upper neighbour");
  SANA_REQUIRE(!lower || last_row, "sana_halo_exchange: last_row required with a lower neighbour");
  SANA_REQUIRE(aligned16(mine) && (!upper || aligned16(upper)) && (!lower || aligned16(lower)) &&
                   (!first_row || aligned16(first_row)) && (!last_row || aligned16(last_row)),
               "sana_halo_exchange: pointers must be 16-byte aligned");
  HaloArgs a;
  a.first_row = static_cast<const uint4*>(first_row);
  a.last_row = static_cast<const uint4*>(last_row);
  a.mine = static_cast<unsigned char*>(mine);
  a.upper = static_cast<unsigned char*>(upper);
  a.lower = static_cast<unsigned char*>(lower);
  a.row_vecs = row_bytes / 16;
  a.step = step;
  a.wait_limit_ns = exchange_wait_limit_ns();
  int64_t blocks = ceil_div(a.row_vecs, 256 * 4);
  // only the block that finishes its copy last waits for the peers (the others exit), so the grid need not be
  // resident at once; a conv row (a few MB at most) is latency-bound on 64 blocks, a whole frame takes more
  const int64_t cap = row_bytes > (4 << 20) ? 2 * sm_count() : 64;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  halo_exchange_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  SANA_LAUNCH_CHECK("halo_exchange kernel");
  return SANA_OK;
}
