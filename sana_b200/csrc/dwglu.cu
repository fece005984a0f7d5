// 3x3 depthwise conv + bias + SiLU-GLU over channels-last image rows (the Mix-FFN middle).
//
// bf16 kernel: a CTA owns a tile of 16 columns x 64 value channels (+ their 64 gate
// channels) and marches down a segment of rows.  Each input row tile (with a one-column
// halo, zero-filled at image edges) is staged once in shared memory by 16-byte cp.async
// through a 10-deep ring (one CTA barrier per two rows); a lane owns one pair of value
// channels and the gate pair of the same index at two neighbouring columns, reads the four
// input columns their windows share from shared memory and feeds three rolling fp32
// accumulators per output (rows y-1, y, y+1) with packed f32x2 FMAs; every input element is
// read from global memory once per CTA, and the GLU needs no exchange between lanes.
#include "common.cuh"

namespace sana {

constexpr int DW_TW = 16;      // output columns per CTA
constexpr int DW_CV = 8;       // 8-channel vectors per role per CTA
constexpr int DW_STAGES = 10;  // ring depth (input rows in flight)
constexpr int DW_THREADS = 256;
constexpr int DW_ROW_CHUNKS = (DW_TW + 2) * 2 * DW_CV;  // 16-byte chunks per staged row = 288
constexpr int DW_STAGE_BYTES = DW_ROW_CHUNKS * 16;

__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr, bool valid) {
  const int sz = valid ? 16 : 0;  // src-size 0 => 16 bytes of zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float fast_silu(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

struct DwArgs {
  const __nv_bfloat16* u;
  const __nv_bfloat16* halo_top;
  const __nv_bfloat16* halo_bot;
  const __nv_bfloat16* weight;  // [2*hid, 9]
  const __nv_bfloat16* bias;    // [2*hid] or null
  __nv_bfloat16* out;
  int rows, W, H, hid, seg_rows;
  int64_t row0;
};

// packed fp32x2 helpers on 64-bit registers (one instruction per two lanes of math)
typedef unsigned long long u64;
__device__ __forceinline__ u64 f2_pack(float lo, float hi) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(u64 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 f2_fma(u64 a, u64 b, u64 c) {
  u64 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ u64 f2_add(u64 a, u64 b) {
  u64 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// two bf16 in one 32-bit word -> packed (fp32, fp32)
__device__ __forceinline__ u64 bf2_to_f2(uint32_t v) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(v << 16), "r"(v & 0xffff0000u));
  return r;
}

__global__ void __launch_bounds__(DW_THREADS, 2) dwconv_glu_bf16_kernel(const DwArgs p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // a lane owns one pair of value channels and the gate pair of the same index, at two
  // neighbouring columns (x, x+1): the 3x3 window of both outputs shares 4 input columns
  const int x0 = blockIdx.y * DW_TW;
  const int x = x0 + 2 * warp;
  const int ys = blockIdx.z * p.seg_rows;
  const int ye = min(p.rows, ys + p.seg_rows);
  const int C2 = 2 * p.hid;
  const int c0 = blockIdx.x * (DW_CV * 8) + lane * 2;  // first of this lane's 2 value channels
  const bool ch_ok = c0 < p.hid;
  const bool ok0 = ch_ok && (x < p.W), ok1 = ch_ok && (x + 1 < p.W);
  const int cw = min(c0, p.hid - 2);

  // taps as packed pairs: w2[tap][0] = value channels (c, c+1), w2[tap][1] = gate channels
  u64 w2[9][2];
  u64 bv[2];
  {
    const __nv_bfloat16* wv = p.weight + (int64_t)cw * 9;
    const __nv_bfloat16* wg = p.weight + (int64_t)(p.hid + cw) * 9;
#pragma unroll
    for (int tap = 0; tap < 9; ++tap) {
      w2[tap][0] = f2_pack(__bfloat162float(wv[tap]), __bfloat162float(wv[9 + tap]));
      w2[tap][1] = f2_pack(__bfloat162float(wg[tap]), __bfloat162float(wg[9 + tap]));
    }
    if (p.bias) {
      bv[0] = f2_pack(__bfloat162float(p.bias[cw]), __bfloat162float(p.bias[cw + 1]));
      bv[1] = f2_pack(__bfloat162float(p.bias[p.hid + cw]), __bfloat162float(p.bias[p.hid + cw + 1]));
    } else {
      bv[0] = bv[1] = 0ull;
    }
  }

  // input-row slots k = 0 .. nin-1  <->  local rows ys-1 .. ye; the first and last slot exist
  // only when that row lies in the same frame as its neighbour inside the segment
  const int nin = ye - ys + 2;
  const int fr_top = (int)((p.row0 + ys + p.H - 1) % p.H);  // frame row of local row ys-1
  const bool need_top = fr_top != p.H - 1;
  const bool need_bot = (int)((p.row0 + ye) % p.H) != 0;
  const int64_t row_elems = (int64_t)p.W * C2;
  const __nv_bfloat16* top_ptr = !need_top ? nullptr : (ys > 0 ? p.u + (int64_t)(ys - 1) * row_elems : p.halo_top);
  const __nv_bfloat16* bot_ptr = !need_bot ? nullptr : (ye < p.rows ? p.u + (int64_t)ye * row_elems : p.halo_bot);
  const __nv_bfloat16* mid_ptr = p.u + (int64_t)ys * row_elems;  // slot 1

  // this thread's (at most two) 16-byte chunks of a staged row: fixed offsets, computed once
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
  const int nvec = p.hid >> 3;
  int64_t src_off[2];
  uint32_t dst_off[2];
  bool src_ok[2], has[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int q = tid + i * DW_THREADS;
    has[i] = q < DW_ROW_CHUNKS;
    const int px = q >> 4, rem = q & 15, rl = rem >> 3, c = rem & 7;
    const int gx = x0 - 1 + px;
    const int gv = blockIdx.x * DW_CV + c;
    src_ok[i] = has[i] && (gx >= 0) && (gx < p.W) && (gv < nvec);
    src_off[i] = src_ok[i] ? (int64_t)gx * C2 + rl * p.hid + (gv << 3) : 0;
    dst_off[i] = q * 16;
  }

  auto issue_row = [&](int k) {
    if (k < nin) {
      const __nv_bfloat16* rp = (k == 0) ? top_ptr : ((k == nin - 1) ? bot_ptr : mid_ptr + (int64_t)(k - 1) * row_elems);
      if (rp != nullptr) {
        const uint32_t sbase = smem_base + (k % DW_STAGES) * DW_STAGE_BYTES;
        cp_async_16(sbase + dst_off[0], rp + src_off[0], src_ok[0]);
        if (has[1]) cp_async_16(sbase + dst_off[1], rp + src_off[1], src_ok[1]);
      }
    }
    cp_async_commit();
  };

  u64 acc[3][2][2];  // [output-row slot][column x / x+1][value / gate]
#pragma unroll
  for (int s = 0; s < 3; ++s)
#pragma unroll
    for (int xo = 0; xo < 2; ++xo) acc[s][xo][0] = acc[s][xo][1] = 0ull;

#pragma unroll 1
  for (int k = 0; k < DW_STAGES - 2; ++k) issue_row(k);

  int fr = fr_top;  // frame row of the input row of the current slot
  __nv_bfloat16* out_ptr = p.out + ((int64_t)(ys - 2) * p.W + x) * p.hid + c0;  // output row of slot k is ys-2+k
  // byte offset of this lane's value word of staged pixel 2*warp (= column x-1), role 0
  const uint32_t rd_off = (uint32_t)(2 * warp * 256 + lane * 4);

  // One step: consume input slot k (local row r = ys-1+k).  PREV/CUR/NEXT are the accumulator
  // slots of output rows (r-1, r, r+1); they rotate with k so no register moves are needed.
  // The CTA synchronises once per two rows (on even k).
  auto step = [&](int k, auto PREVc, auto CURc, auto NEXTc) {
    constexpr int PREV = decltype(PREVc)::value, CUR = decltype(CURc)::value, NEXT = decltype(NEXTc)::value;
    if ((k & 1) == 0) {
      cp_async_wait<DW_STAGES - 4>();  // rows k and k+1 have landed (for this thread's copies)
      __syncthreads();                 // ... for everybody's; and rows k-2, k-1 are no longer read
      issue_row(k + DW_STAGES - 2);
      issue_row(k + DW_STAGES - 1);
    }
    const bool first = (k == 0), last = (k == nin - 1);
    const bool have = first ? need_top : (last ? need_bot : true);
    if (have) {
      const unsigned char* sp = smem + (k % DW_STAGES) * DW_STAGE_BYTES + rd_off;
      u64 col[4][2];  // input columns x-1 .. x+2, [value / gate]
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        col[c][0] = bf2_to_f2(*reinterpret_cast<const uint32_t*>(sp + c * 256));
        col[c][1] = bf2_to_f2(*reinterpret_cast<const uint32_t*>(sp + c * 256 + 128));
      }
      // input row r is the row BELOW output r-1 (taps 6..8), the centre of output r (taps 3..5)
      // and the row ABOVE output r+1 (taps 0..2); vertical neighbours must share the frame.
      if (k >= 2 && fr != 0) {  // output r-1 is inside the segment
#pragma unroll
        for (int xo = 0; xo < 2; ++xo)
#pragma unroll
          for (int dx = 0; dx < 3; ++dx)
#pragma unroll
            for (int h = 0; h < 2; ++h) acc[PREV][xo][h] = f2_fma(w2[6 + dx][h], col[xo + dx][h], acc[PREV][xo][h]);
      }
      if (!first && !last) {
#pragma unroll
        for (int xo = 0; xo < 2; ++xo)
#pragma unroll
          for (int dx = 0; dx < 3; ++dx)
#pragma unroll
            for (int h = 0; h < 2; ++h) acc[CUR][xo][h] = f2_fma(w2[3 + dx][h], col[xo + dx][h], acc[CUR][xo][h]);
      }
      if (k + 2 < nin && fr != p.H - 1) {  // output r+1 is inside the segment
#pragma unroll
        for (int xo = 0; xo < 2; ++xo)
#pragma unroll
          for (int dx = 0; dx < 3; ++dx)
#pragma unroll
            for (int h = 0; h < 2; ++h) acc[NEXT][xo][h] = f2_fma(w2[dx][h], col[xo + dx][h], acc[NEXT][xo][h]);
      }
    }
    if (k >= 2) {  // output row r-1 = ys + k - 2 is complete
#pragma unroll
      for (int xo = 0; xo < 2; ++xo) {
        float a0, a1, g0, g1;
        f2_unpack(f2_add(acc[PREV][xo][0], bv[0]), a0, a1);
        f2_unpack(f2_add(acc[PREV][xo][1], bv[1]), g0, g1);
        if (xo == 0 ? ok0 : ok1)
          *reinterpret_cast<uint32_t*>(out_ptr + xo * p.hid) = pack_bf16(a0 * fast_silu(g0), a1 * fast_silu(g1));
      }
    }
#pragma unroll
    for (int xo = 0; xo < 2; ++xo) acc[PREV][xo][0] = acc[PREV][xo][1] = 0ull;  // becomes NEXT of the next step
    out_ptr += (int64_t)p.W * p.hid;
    fr = (fr + 1 == p.H) ? 0 : fr + 1;
  };

  using I0 = std::integral_constant<int, 0>;
  using I1 = std::integral_constant<int, 1>;
  using I2 = std::integral_constant<int, 2>;
  // six slots per trip so that both the accumulator rotation (period 3) and the barrier
  // cadence (period 2) are compile-time
#pragma unroll 1
  for (int k = 0; k < nin; k += 6) {
    step(k, I0{}, I1{}, I2{});
    if (k + 1 < nin) step(k + 1, I1{}, I2{}, I0{});
    if (k + 2 < nin) step(k + 2, I2{}, I0{}, I1{});
    if (k + 3 < nin) step(k + 3, I0{}, I1{}, I2{});
    if (k + 4 < nin) step(k + 4, I1{}, I2{}, I0{});
    if (k + 5 < nin) step(k + 5, I2{}, I0{}, I1{});
  }
  cp_async_wait<0>();
}

// Plain fp32 version (parity path): one thread per (row, x, channel pair value/gate).
__global__ void dwconv_glu_f32_kernel(const float* __restrict__ u, const float* __restrict__ halo_top,
                                      const float* __restrict__ halo_bot, const float* __restrict__ weight,
                                      const float* __restrict__ bias, float* __restrict__ out, int rows, int W, int H,
                                      int hid, int64_t row0) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)rows * W * hid;
  if (idx >= total) return;
  const int c = (int)(idx % hid);
  const int x = (int)((idx / hid) % W);
  const int r = (int)(idx / ((int64_t)hid * W));
  const int C2 = 2 * hid;
  const int fr = (int)((row0 + r) % H);
  float acc[2];
#pragma unroll
  for (int role = 0; role < 2; ++role) {
    const int chn = role * hid + c;
    float s = bias ? bias[chn] : 0.f;
    for (int dy = -1; dy <= 1; ++dy) {
      if ((dy < 0 && fr == 0) || (dy > 0 && fr == H - 1)) continue;
      const int rr = r + dy;
      const float* rp = rr < 0 ? halo_top : (rr >= rows ? halo_bot : u + (int64_t)rr * W * C2);
      for (int dx = -1; dx <= 1; ++dx) {
        const int xx = x + dx;
        if (xx < 0 || xx >= W) continue;
        s = fmaf(weight[chn * 9 + (dy + 1) * 3 + (dx + 1)], rp[(int64_t)xx * C2 + chn], s);
      }
    }
    acc[role] = s;
  }
  out[idx] = acc[0] * (acc[1] / (1.0f + expf(-acc[1])));
}

}  // namespace sana

using namespace sana;

extern "C" int sana_dwconv_glu(const void* u, const void* halo_top, const void* halo_bot, const void* weight,
                               const void* bias, void* out, int64_t rows, int64_t W, int64_t H, int64_t row0,
                               int64_t hid, int dtype, void* stream) {
  SANA_REQUIRE(u && weight && out, "sana_dwconv_glu: null pointer");
  SANA_REQUIRE(rows > 0 && W > 0 && H > 0 && hid > 0 && row0 >= 0, "sana_dwconv_glu: sizes must be positive");
  SANA_REQUIRE(hid % 8 == 0, "sana_dwconv_glu: hid must be a multiple of 8");
  SANA_REQUIRE(rows < (1 << 24) && W < (1 << 20) && hid < (1 << 20), "sana_dwconv_glu: size out of range");
  SANA_REQUIRE((row0 % H == 0) || halo_top, "sana_dwconv_glu: halo_top required (first row is inside a frame)");
  SANA_REQUIRE(((row0 + rows) % H == 0) || halo_bot, "sana_dwconv_glu: halo_bot required (last row is inside a frame)");
  SANA_REQUIRE(aligned16(u) && aligned16(out) && (!halo_top || aligned16(halo_top)) &&
                   (!halo_bot || aligned16(halo_bot)),
               "sana_dwconv_glu: pointers must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == SANA_BF16) {
    DwArgs a;
    a.u = static_cast<const __nv_bfloat16*>(u);
    a.halo_top = static_cast<const __nv_bfloat16*>(halo_top);
    a.halo_bot = static_cast<const __nv_bfloat16*>(halo_bot);
    a.weight = static_cast<const __nv_bfloat16*>(weight);
    a.bias = static_cast<const __nv_bfloat16*>(bias);
    a.out = static_cast<__nv_bfloat16*>(out);
    a.rows = (int)rows, a.W = (int)W, a.H = (int)H, a.hid = (int)hid, a.row0 = row0;
    const int64_t gx = ceil_div(hid / 8, DW_CV), gy = ceil_div(W, DW_TW);
    // rows per CTA: long segments amortise the two halo rows; shorten them until the grid
    // covers the device a few times over.
    int seg = 32;
    while (seg > 4 && gx * gy * ceil_div(rows, seg) < 4 * (int64_t)sm_count()) seg >>= 1;
    a.seg_rows = seg;
    const int64_t gz = ceil_div(rows, seg);
    SANA_REQUIRE(gy < 65536 && gz < 65536, "sana_dwconv_glu: grid too large");
    static bool attr_set = false;
    const int smem_bytes = DW_STAGES * DW_STAGE_BYTES;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(dwconv_glu_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
      if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(dwconv_glu)");
      attr_set = true;
    }
    dwconv_glu_bf16_kernel<<<dim3((unsigned)gx, (unsigned)gy, (unsigned)gz), DW_THREADS, smem_bytes, st>>>(a);
  } else if (dtype == SANA_F32) {
    const int64_t total = rows * W * hid;
    dwconv_glu_f32_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(
        static_cast<const float*>(u), static_cast<const float*>(halo_top), static_cast<const float*>(halo_bot),
        static_cast<const float*>(weight), static_cast<const float*>(bias), static_cast<float*>(out), (int)rows, (int)W,
        (int)H, (int)hid, row0);
  } else {
    return fail(SANA_ERR_UNSUPPORTED, "sana_dwconv_glu: unsupported dtype %d", dtype);
  }
  SANA_LAUNCH_CHECK("dwconv_glu kernel");
  return SANA_OK;
}
