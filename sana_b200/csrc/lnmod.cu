// adaLN-single LayerNorm + modulate: one warp per token row, the row held in registers
// (packed, as loaded) so global memory is read once and written once; the per-sample
// modulation vectors are combined once per block into shared memory.
#include "fp4_quant.cuh"

namespace sana {

template <typename T>
struct Vec16;  // 16-byte vector of T
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void unpack(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x), f[1] = bf16_hi(v.x), f[2] = bf16_lo(v.y), f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z), f[5] = bf16_hi(v.z), f[6] = bf16_lo(v.w), f[7] = bf16_hi(v.w);
  }
  __device__ static uint4 pack(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
  }
};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x), f[1] = __uint_as_float(v.y), f[2] = __uint_as_float(v.z), f[3] = __uint_as_float(v.w);
  }
  __device__ static uint4 pack(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Shared memory holds, for the batch sample being processed, the two fp32 modulation vectors
// mul = 1 + (t[scale_row] + table[scale_row]) and add = t[shift_row] + table[shift_row], laid
// out as planes of float4 (plane p holds elements 4p..4p+3 of every 16-byte vector) so that a
// warp's reads are conflict-free. A block owns a contiguous range of rows and restages the
// vectors when the range crosses into the next sample.
// With FP4 (bf16 only) the kernel also - or only, when z is null - writes the NVFP4 image of its output: the
// modulated row is rounded to bf16 exactly as it would be stored, then quantised 16 channels at a time (two
// neighbouring lanes hold a block) with the tensor scale given by the caller; the largest magnitude produced is
// accumulated into sink.amax_out.
template <typename T, int MAXV, bool FP4>
__global__ void __launch_bounds__(256)
ln_modulate_kernel(const T* __restrict__ x, const T* __restrict__ table, const T* __restrict__ t, T* __restrict__ z,
                   int64_t rows, int N, int C, int tb_shift, int tb_scale, int t_rows, int t_shift, int t_scale,
                   float eps, int rows_per_block, const Fp4Sink sink) {
  constexpr int VN = Vec16<T>::N;
  constexpr int PLANES = VN / 4;
  extern __shared__ float4 ln_smem[];
  const int nvec = C / VN;
  float4* s_mul = ln_smem;                  // [PLANES][nvec]
  float4* s_add = ln_smem + PLANES * nvec;  // [PLANES][nvec]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarp = blockDim.x >> 5;
  const int64_t row0 = (int64_t)blockIdx.x * rows_per_block;
  const int64_t row1 = (row0 + rows_per_block < rows) ? row0 + rows_per_block : rows;
  if (row0 >= row1) return;
  const float inv_c = 1.0f / (float)C;
  const float ts = FP4 ? __ldg(sink.scale_in + 1) : 0.f;
  const float inv6ts = FP4 ? __frcp_rn(6.0f * ts) : 0.f;
  float amax_local = 0.f;
  for (int64_t b = row0 / N; b * N < row1; ++b) {
    const int64_t seg0 = (b * N > row0) ? b * N : row0;
    const int64_t seg1 = ((b + 1) * N < row1) ? (b + 1) * N : row1;
    __syncthreads();  // every warp is done with the previous sample's vectors
    {
      const T* tsc = t + (b * t_rows + t_scale) * C;
      const T* tsh = t + (b * t_rows + t_shift) * C;
      const T* bsc = table + (int64_t)tb_scale * C;
      const T* bsh = table + (int64_t)tb_shift * C;
      float* fm = reinterpret_cast<float*>(s_mul);
      float* fa = reinterpret_cast<float*>(s_add);
      for (int i = threadIdx.x; i < C; i += blockDim.x) {
        const int v = i / VN, e = i % VN;
        const int slot = ((e >> 2) * nvec + v) * 4 + (e & 3);
        fm[slot] = 1.0f + (to_float(tsc[i]) + to_float(bsc[i]));
        fa[slot] = to_float(tsh[i]) + to_float(bsh[i]);
      }
    }
    __syncthreads();
    auto load = [&](uint4 (&raw)[MAXV], int64_t row) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) raw[i] = ldg_nc_u4(xr + v);
      }
    };
    auto process = [&](const uint4 (&raw)[MAXV], int64_t row) {
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          float f[VN];
          Vec16<T>::unpack(raw[i], f);
#pragma unroll
          for (int e = 0; e < VN; ++e) sum += f[e];
        }
      }
      const float mean = warp_sum(sum) * inv_c;
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          float f[VN];
          Vec16<T>::unpack(raw[i], f);
#pragma unroll
          for (int e = 0; e < VN; ++e) {
            const float d = f[e] - mean;
            sq = fmaf(d, d, sq);
          }
        }
      }
      const float rstd = rsqrtf(warp_sum(sq) * inv_c + eps);
      uint4* zr = reinterpret_cast<uint4*>(z + row * C);
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int v = lane + 32 * i;
        const bool in = v < nvec;
        uint4 packed = make_uint4(0u, 0u, 0u, 0u);
        if (in) {
          float f[VN];
          Vec16<T>::unpack(raw[i], f);
#pragma unroll
          for (int p = 0; p < PLANES; ++p) {
            const float4 m = s_mul[p * nvec + v];
            const float4 a = s_add[p * nvec + v];
            f[4 * p + 0] = fmaf((f[4 * p + 0] - mean) * rstd, m.x, a.x);
            f[4 * p + 1] = fmaf((f[4 * p + 1] - mean) * rstd, m.y, a.y);
            f[4 * p + 2] = fmaf((f[4 * p + 2] - mean) * rstd, m.z, a.z);
            f[4 * p + 3] = fmaf((f[4 * p + 3] - mean) * rstd, m.w, a.w);
          }
          packed = Vec16<T>::pack(f);
          if (!FP4 || z != nullptr) zr[v] = packed;
        }
        if (FP4 && 32 * i < nvec) {  // warp-uniform: some lane of this round holds channels (bf16: VN = 8)
          float fq[8];
          fq[0] = bf16_lo(packed.x), fq[1] = bf16_hi(packed.x), fq[2] = bf16_lo(packed.y), fq[3] = bf16_hi(packed.y);
          fq[4] = bf16_lo(packed.z), fq[5] = bf16_hi(packed.z), fq[6] = bf16_lo(packed.w), fq[7] = bf16_hi(packed.w);
#pragma unroll
          for (int e = 0; e < 8; ++e) amax_local = fmaxf(amax_local, fabsf(fq[e]));
          uint32_t sb;
          const uint32_t codes = fp4_quant8_of16(fq, ts, inv6ts, &sb);
          if (in) *reinterpret_cast<uint32_t*>(sink.q + row * (int64_t)(C >> 1) + 4 * v) = codes;
          // the four block scales of a 64-channel tile sit in the even lanes of a group of eight
          if (!in) sb = 0u;
          const uint32_t s1 = __shfl_down_sync(0xffffffffu, sb, 2), s2 = __shfl_down_sync(0xffffffffu, sb, 4),
                         s3 = __shfl_down_sync(0xffffffffu, sb, 6);
          if (in && (lane & 7) == 0) {
            const int64_t tile = (row >> 7) * sink.ktiles4 + (v >> 3);
            *reinterpret_cast<uint32_t*>(sink.sf + tile * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4) =
                sb | (s1 << 8) | (s2 << 16) | (s3 << 24);
          }
        }
      }
    };
    // two register sets in ping-pong: the next row's loads are in flight while this row is
    // reduced, modulated and stored
    uint4 ra[MAXV], rb[MAXV];
    int64_t row = seg0 + warp;
    if (row < seg1) load(ra, row);
    for (; row < seg1; row += 2 * nwarp) {
      const int64_t r1 = row + nwarp, r2 = row + 2 * nwarp;
      if (r1 < seg1) load(rb, r1);
      process(ra, row);
      if (r2 < seg1) load(ra, r2);
      if (r1 < seg1) process(rb, r1);
    }
  }
  if (FP4 && sink.amax_out != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax_local = fmaxf(amax_local, __shfl_xor_sync(0xffffffffu, amax_local, o));
    if (lane == 0) atomicMax(reinterpret_cast<unsigned int*>(sink.amax_out), __float_as_uint(amax_local));  // >= 0
  }
}

template <typename T, bool FP4>
static int launch_ln(const void* x, const void* table, const void* t, void* z, int64_t B, int64_t N, int64_t C,
                     int tb_shift, int tb_scale, int t_rows, int t_shift, int t_scale, float eps, cudaStream_t st,
                     const Fp4Sink& sink) {
  const int64_t rows = B * N;
  const int nvec = (int)(C / Vec16<T>::N);
  const int per_lane = (nvec + 31) / 32;
  const size_t smem = (size_t)2 * C * sizeof(float);
  const T* xp = static_cast<const T*>(x);
  const T* tb = static_cast<const T*>(table);
  const T* tp = static_cast<const T*>(t);
  T* zp = static_cast<T*>(z);
#define SANA_LN_CASE(MV)                                                                                       \
  if (per_lane <= MV) {                                                                                        \
    if (smem > 48 * 1024) {                                                                                    \
      cudaError_t e = cudaFuncSetAttribute(ln_modulate_kernel<T, MV, FP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                         \
      if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(ln_modulate)");                       \
    }                                                                                                          \
    /* one wave of blocks (as many as are resident), each over a contiguous range of rows */                  \
    int per_sm = 0;                                                                                            \
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ln_modulate_kernel<T, MV, FP4>, 256, smem) !=        \
            cudaSuccess || per_sm < 1) {                                                                       \
      cudaGetLastError();                                                                                      \
      per_sm = 1;                                                                                              \
    }                                                                                                          \
    int64_t rpb = ceil_div(rows, (int64_t)sm_count() * per_sm);                                                \
    rpb = ceil_div(rpb, 8) * 8;                                                                                \
    const unsigned grid = (unsigned)ceil_div(rows, rpb);                                                       \
    ln_modulate_kernel<T, MV, FP4><<<grid, 256, smem, st>>>(xp, tb, tp, zp, rows, (int)N, (int)C, tb_shift, tb_scale,   \
                                                       t_rows, t_shift, t_scale, eps, (int)rpb, sink);         \
    SANA_LAUNCH_CHECK("ln_modulate kernel");                                                                   \
    return SANA_OK;                                                                                            \
  }
  SANA_LN_CASE(5)
  SANA_LN_CASE(9)
  SANA_LN_CASE(16)
  SANA_LN_CASE(32)
#undef SANA_LN_CASE
  return fail(SANA_ERR_UNSUPPORTED, "sana_ln_modulate: C=%lld too large", (long long)C);
}

}  // namespace sana

using namespace sana;

extern "C" int sana_ln_modulate_rows(const void* x, const void* table, const void* t, void* z, int64_t B, int64_t N,
                                     int64_t C, int table_rows, int table_shift_row, int table_scale_row, int t_rows,
                                     int t_shift_row, int t_scale_row, float eps, int dtype, void* stream) {
  SANA_REQUIRE(x && table && t && z, "sana_ln_modulate: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && C > 0, "sana_ln_modulate: sizes must be positive");
  SANA_REQUIRE(C % 8 == 0 && C * (dtype == SANA_F32 ? 4 : 2) <= 16384,
               "sana_ln_modulate: C must be a multiple of 8 and a row at most 16 KiB");
  SANA_REQUIRE(table_rows > 0 && table_shift_row >= 0 && table_shift_row < table_rows && table_scale_row >= 0 &&
                   table_scale_row < table_rows,
               "sana_ln_modulate: bad table row");
  SANA_REQUIRE(t_rows > 0 && t_shift_row >= 0 && t_shift_row < t_rows && t_scale_row >= 0 && t_scale_row < t_rows,
               "sana_ln_modulate: bad row of t");
  SANA_REQUIRE(aligned16(x) && aligned16(table) && aligned16(t) && aligned16(z),
               "sana_ln_modulate: pointers must be 16-byte aligned");
  SANA_REQUIRE(B * N < ((int64_t)1 << 31) * 8, "sana_ln_modulate: too many rows");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const Fp4Sink none = {};
  if (dtype == SANA_BF16)
    return launch_ln<__nv_bfloat16, false>(x, table, t, z, B, N, C, table_shift_row, table_scale_row, t_rows, t_shift_row,
                                           t_scale_row, eps, st, none);
  if (dtype == SANA_F32)
    return launch_ln<float, false>(x, table, t, z, B, N, C, table_shift_row, table_scale_row, t_rows, t_shift_row,
                                   t_scale_row, eps, st, none);
  return fail(SANA_ERR_UNSUPPORTED, "sana_ln_modulate: unsupported dtype %d", dtype);
}

extern "C" int sana_ln_modulate(const void* x, const void* table, const void* t, void* z, int64_t B, int64_t N,
                                int64_t C, int shift_row, int scale_row, float eps, int dtype, void* stream) {
  return sana_ln_modulate_rows(x, table, t, z, B, N, C, 6, shift_row, scale_row, 6, shift_row, scale_row, eps, dtype,
                               stream);
}

extern "C" int sana_ln_modulate_fp4(const void* x, const void* table, const void* t, void* z, void* q, void* sf,
                                    const float* scale_in, float* amax_out, int64_t B, int64_t N, int64_t C, int shift_row,
                                    int scale_row, float eps, void* stream) {
  SANA_REQUIRE(x && table && t && q && sf && scale_in, "sana_ln_modulate_fp4: null pointer");
  SANA_REQUIRE(B > 0 && N > 0 && C > 0, "sana_ln_modulate_fp4: sizes must be positive");
  SANA_REQUIRE(C % 32 == 0 && C * 2 <= 16384, "sana_ln_modulate_fp4: C must be a multiple of 32 and a row at most 16 KiB");
  SANA_REQUIRE(shift_row >= 0 && shift_row < 6 && scale_row >= 0 && scale_row < 6, "sana_ln_modulate_fp4: bad table row");
  SANA_REQUIRE(aligned16(x) && aligned16(table) && aligned16(t) && (!z || aligned16(z)) && aligned16(q) && aligned16(sf),
               "sana_ln_modulate_fp4: pointers must be 16-byte aligned");
  SANA_REQUIRE(B * N < ((int64_t)1 << 31) * 8, "sana_ln_modulate_fp4: too many rows");
  Fp4Sink sink;
  sink.q = static_cast<unsigned char*>(q);
  sink.sf = static_cast<unsigned char*>(sf);
  sink.scale_in = scale_in;
  sink.amax_out = amax_out;
  sink.K = (int)C;
  sink.ktiles4 = (int)ktiles4_of(C);
  return launch_ln<__nv_bfloat16, true>(x, table, t, z, B, N, C, shift_row, scale_row, 6, shift_row, scale_row, eps,
                                        static_cast<cudaStream_t>(stream), sink);
}
