// 3x3 depthwise conv + bias + SiLU-GLU over channels-last image rows (the Mix-FFN middle).
//
// bf16 kernel: every warp is an independent worker.  It owns two neighbouring output columns
// x, x+1 and 64 value channels (+ the 64 gate channels of the same index; a lane owns one
// channel pair of each) and marches down a segment of rows.  Per input row it needs the four
// pixels x-1 .. x+2 of both channel groups: one 1 KiB box of a 4-D tensor map
// {channel, value/gate, x, row}, fetched by a bulk-tensor copy into the warp's own ring of
// DW_STAGES boxes in shared memory (image borders come back as zeros from the out-of-range
// fill).  Lane 0 refills a box as soon as the warp has consumed it, so there is no CTA-wide
// barrier and no per-thread address arithmetic in the row loop.  Each loaded row feeds three
// rolling fp32 accumulators per output (rows y-1, y, y+1) with packed f32x2 FMAs; the GLU
// needs no exchange between lanes.  Neighbouring warps load overlapping pixels, which costs
// L2 bandwidth but no DRAM traffic.
#include "tc_common.cuh"

namespace sana {

__device__ int g_dw_status = 0;  // soft-error word: 1 = a wait on an input row timed out

constexpr int DW_WARPS = 8;  // single-warp CTAs measured 30 % slower
constexpr int DW_TW = 2 * DW_WARPS;  // output columns per CTA (two per warp)
constexpr int DW_THREADS = 32 * DW_WARPS;
constexpr int DW_CTAS_PER_SM = 16 / DW_WARPS;  // 16 resident warps (register-limited)
constexpr int DW_CH = 64;       // value channels per warp (and as many gate channels)
constexpr int DW_STAGES = 9;    // input rows in flight per warp
constexpr int DW_SLOTS = DW_STAGES / 3;  // the ring is filled and drained three rows at a time
constexpr int DW_BOX_BYTES = 4 * 2 * DW_CH * 2;  // 4 pixels x {value, gate} x 64 channels x bf16 = 1 KiB
constexpr int DW_RING_BYTES = DW_WARPS * DW_STAGES * DW_BOX_BYTES;
constexpr int DW_SMEM_BYTES = DW_RING_BYTES + DW_WARPS * DW_STAGES * 8;

__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Bounded wait for an input row.  On time-out the warp records the soft error, gives copies
// that may still be in flight towards its ring time to land (the CTA's shared memory must not
// be handed to another block under them) and exits; warps are independent, so nobody waits
// for it.  Not returning a flag keeps the row loop free of per-step liveness checks.
__device__ __forceinline__ void dw_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait_poll(bar, parity)) return;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait_poll(bar, parity)) {
    if ((++spins & 1023u) == 0 && clock64() - t0 > TC_WAIT_LIMIT_CYCLES) {
      atomicExch(&g_dw_status, 1);
      const long long t1 = clock64();
      while (clock64() - t1 < 2000000LL) {
      }
      asm volatile("exit;");
    }
  }
}

struct DwArgs {
  const __nv_bfloat16* weight;  // [2*hid, 9]
  const __nv_bfloat16* bias;    // [2*hid] or null
  __nv_bfloat16* out;
  int rows, W, H, hid, seg_rows;
  int64_t row0;
  float* amax_out;  // when set: atomically raised to the largest |output| (as stored, bf16)
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
__device__ __forceinline__ u64 f2_mul(u64 a, u64 b) {
  u64 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// two bf16 in one 32-bit word -> packed (fp32, fp32)
__device__ __forceinline__ u64 bf2_to_f2(uint32_t v) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(v << 16), "r"(v & 0xffff0000u));
  return r;
}
__device__ __forceinline__ float tanh_fast(float x) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// a * silu(g) on a channel pair; silu(g) = h + h * tanh(h) with h = g / 2 (one MUFU op per element)
__device__ __forceinline__ uint32_t glu_pair(u64 a2, u64 g2) {
  const u64 h2 = f2_mul(g2, f2_pack(0.5f, 0.5f));
  float h0, h1, o0, o1;
  f2_unpack(h2, h0, h1);
  const u64 s2 = f2_fma(h2, f2_pack(tanh_fast(h0), tanh_fast(h1)), h2);
  f2_unpack(f2_mul(a2, s2), o0, o1);
  return pack_bf16(o0, o1);
}

__global__ void __launch_bounds__(DW_THREADS, DW_CTAS_PER_SM)
dwconv_glu_bf16_kernel(const __grid_constant__ CUtensorMap tmU3, const __grid_constant__ CUtensorMap tmU,
                       const __grid_constant__ CUtensorMap tmTop, const __grid_constant__ CUtensorMap tmBot,
                       const DwArgs p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int x = blockIdx.y * DW_TW + 2 * warp;  // this warp's columns: x, x + 1
  if (x >= p.W) return;                         // warps are independent: no CTA-wide barrier below
  const int ys = blockIdx.z * p.seg_rows;
  const int ye = min(p.rows, ys + p.seg_rows);
  const int cbase = blockIdx.x * DW_CH;
  const int c0 = cbase + lane * 2;  // first of this lane's 2 value channels
  const bool ok0 = c0 < p.hid, ok1 = ok0 && (x + 1 < p.W);
  const int cw = min(c0, p.hid - 2);

  const uint32_t ring = smem_u32(smem) + (uint32_t)(warp * DW_STAGES * DW_BOX_BYTES);
  // the ring is refilled in slots of three rows (one trip of the row loop), one barrier per slot
  const uint32_t bars = smem_u32(smem) + (uint32_t)(DW_RING_BYTES + warp * DW_STAGES * 8);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < DW_SLOTS; ++s) mbar_init(bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // input-row slots k = 0 .. nin-1  <->  local rows ys-1 .. ye; the first and last slot exist
  // only when that row lies in the same frame as its neighbour inside the segment
  const int nin = ye - ys + 2;
  const int fr_top = (int)((p.row0 + ys + p.H - 1) % p.H);  // frame row of local row ys-1
  const bool need_top = fr_top != p.H - 1;
  const bool need_bot = (int)((p.row0 + ye) % p.H) != 0;

  // does input slot k hold a row? (the halo slots at both ends only inside a frame)
  auto exists = [&](int k) { return k < nin && (k != 0 || need_top) && (k != nin - 1 || need_bot); };
  // lane 0: fetch input slots kk, kk+1, kk+2 into ring slot `slot` (three boxes of 1 KiB).  Rows
  // strictly inside the segment come as one three-row copy; a slot that touches the halo slots
  // is fetched row by row from whichever tensor holds each row.  A slot without any row is never
  // waited for, but its barrier phase is completed all the same so that the parity of later
  // passes stays in step.
  auto refill = [&](int kk, int slot) {
    if (kk >= nin) return;
    const uint32_t bar = bars + 8 * slot, dst = ring + slot * (3 * DW_BOX_BYTES);
    if (kk >= 1 && kk + 2 <= nin - 2) {
      mbar_expect_tx(bar, 3 * DW_BOX_BYTES);
      tma_load_4d(dst, &tmU3, bar, cbase, 0, x - 1, ys - 1 + kk);
      return;
    }
    int n = 0;
    for (int j = 0; j < 3; ++j) n += exists(kk + j) ? 1 : 0;
    if (n == 0) {
      mbar_arrive(bar);
      return;
    }
    mbar_expect_tx(bar, n * DW_BOX_BYTES);
    for (int j = 0; j < 3; ++j) {
      const int k = kk + j;
      if (!exists(k)) continue;
      const CUtensorMap* tm = &tmU;
      int r = ys - 1 + k;
      if (k == 0 && ys == 0) tm = &tmTop, r = 0;
      if (k == nin - 1 && ye >= p.rows) tm = &tmBot, r = 0;
      tma_load_4d(dst + j * DW_BOX_BYTES, tm, bar, cbase, 0, x - 1, r);
    }
  };
  if (lane == 0) {
#pragma unroll 1
    for (int s = 0; s < DW_SLOTS; ++s) refill(3 * s, s);
  }

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

  // [output-row slot][column x / x+1][value / gate].  A slot is (re)started in its NEXT role,
  // where the first tap's FMA takes the bias as its addend.
  u64 acc[3][2][2];
#pragma unroll
  for (int s = 0; s < 3; ++s)
#pragma unroll
    for (int xo = 0; xo < 2; ++xo) acc[s][xo][0] = bv[0], acc[s][xo][1] = bv[1];

  int fr = fr_top;  // frame row of the input row of the current slot
  const uint32_t ring_lane = ring + (uint32_t)(lane * 4);  // this lane's word of pixel x-1, value group, box 0
  const int64_t out_step = (int64_t)p.W * p.hid;
  __nv_bfloat16* out0 = p.out + ((int64_t)(ys - 2) * p.W + x) * p.hid + c0;  // output row of slot k is ys-2+k
  __nv_bfloat16* out1 = out0 + p.hid;

  // input columns x-1 .. x+2 of the box at shared address `b` (this lane's word), [value / gate]
  auto load_cols = [&](uint32_t b, u64 (&col)[4][2]) {
    uint32_t w[8];
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[0]) : "r"(b));
    asm volatile("ld.shared.b32 %0, [%1+128];" : "=r"(w[1]) : "r"(b));
    asm volatile("ld.shared.b32 %0, [%1+256];" : "=r"(w[2]) : "r"(b));
    asm volatile("ld.shared.b32 %0, [%1+384];" : "=r"(w[3]) : "r"(b));
    asm volatile("ld.shared.b32 %0, [%1+512];" : "=r"(w[4]) : "r"(b));
    asm volatile("ld.shared.b32 %0, [%1+640];" : "=r"(w[5]) : "r"(b));
    asm volatile("ld.shared.b32 %0, [%1+768];" : "=r"(w[6]) : "r"(b));
    asm volatile("ld.shared.b32 %0, [%1+896];" : "=r"(w[7]) : "r"(b));
#pragma unroll
    for (int c = 0; c < 4; ++c) col[c][0] = bf2_to_f2(w[2 * c]), col[c][1] = bf2_to_f2(w[2 * c + 1]);
  };
  // taps of kernel row `trow` of the loaded input row into an accumulator slot
  auto taps = [&](u64 (&a)[2][2], const u64 (&col)[4][2], int trow) {
#pragma unroll
    for (int dx = 0; dx < 3; ++dx)
#pragma unroll
      for (int xo = 0; xo < 2; ++xo)
#pragma unroll
        for (int h = 0; h < 2; ++h) a[xo][h] = f2_fma(w2[3 * trow + dx][h], col[xo + dx][h], a[xo][h]);
  };
  auto taps_start = [&](u64 (&a)[2][2], const u64 (&col)[4][2]) {  // kernel row 0, starting from the bias
#pragma unroll
    for (int xo = 0; xo < 2; ++xo)
#pragma unroll
      for (int h = 0; h < 2; ++h) a[xo][h] = f2_fma(w2[0][h], col[xo][h], bv[h]);
#pragma unroll
    for (int dx = 1; dx < 3; ++dx)
#pragma unroll
      for (int xo = 0; xo < 2; ++xo)
#pragma unroll
        for (int h = 0; h < 2; ++h) a[xo][h] = f2_fma(w2[dx][h], col[xo + dx][h], a[xo][h]);
  };
  auto restart = [&](u64 (&a)[2][2]) {
#pragma unroll
    for (int xo = 0; xo < 2; ++xo) a[xo][0] = bv[0], a[xo][1] = bv[1];
  };
  uint32_t amax_bits = 0u;  // running maximum of |output| per 16-bit half (bf16 bit patterns order like integers)
  auto emit = [&](const u64 (&a)[2][2]) {
    const uint32_t o0 = glu_pair(a[0][0], a[0][1]);
    const uint32_t o1 = glu_pair(a[1][0], a[1][1]);
    if (ok0) *reinterpret_cast<uint32_t*>(out0) = o0;
    if (ok1) *reinterpret_cast<uint32_t*>(out1) = o1;
    amax_bits = __vmaxu2(amax_bits, __vmaxu2(ok0 ? (o0 & 0x7fff7fffu) : 0u, ok1 ? (o1 & 0x7fff7fffu) : 0u));
  };
  auto advance = [&]() {
    out0 += out_step;
    out1 += out_step;
    fr = (fr + 1 == p.H) ? 0 : fr + 1;
  };

  // One step consumes input slot k (local row r = ys-1+k) from ring box `slot`.  PREV/CUR/NEXT
  // are the accumulator slots of output rows (r-1, r, r+1); they rotate with k so no register
  // moves are needed.  Input row r is the row BELOW output r-1 (kernel row 2), the centre of
  // output r (kernel row 1) and the row ABOVE output r+1 (kernel row 0); vertical neighbours
  // must share the frame.
  //
  // General step: any k, including the halo slots at both ends of the segment.
  auto step_any = [&](int k, int row_slot, auto PREVc, auto CURc, auto NEXTc) {
    constexpr int PREV = decltype(PREVc)::value, CUR = decltype(CURc)::value, NEXT = decltype(NEXTc)::value;
    const bool first = (k == 0), last = (k == nin - 1);
    const bool have = first ? need_top : (last ? need_bot : true);
    bool started = false;
    if (have) {
      u64 col[4][2];
      load_cols(ring_lane + row_slot * DW_BOX_BYTES, col);
      if (k >= 2 && fr != 0) taps(acc[PREV], col, 2);  // output r-1 is inside the segment
      if (!first && !last) taps(acc[CUR], col, 1);
      if (k + 2 < nin && fr != p.H - 1) {  // output r+1 is inside the segment
        taps_start(acc[NEXT], col);
        started = true;
      }
    }
    if (k >= 2) emit(acc[PREV]);  // output row r-1 = ys + k - 2 is complete
    if (!started) restart(acc[NEXT]);
    advance();
  };
  // Interior step away from frame edges: 2 <= k <= nin-3 and the input row is neither the
  // first nor the last of its frame, so the row exists and all three outputs take it.  One
  // branch-free block - the FMAs, the conversions and the previous row's GLU - which is what
  // lets the few resident warps overlap their fixed-latency dependencies.
  auto step_mid = [&](int row_slot, auto PREVc, auto CURc, auto NEXTc) {
    constexpr int PREV = decltype(PREVc)::value, CUR = decltype(CURc)::value, NEXT = decltype(NEXTc)::value;
    u64 col[4][2];
    load_cols(ring_lane + row_slot * DW_BOX_BYTES, col);
    taps(acc[PREV], col, 2);
    taps(acc[CUR], col, 1);
    taps_start(acc[NEXT], col);
    emit(acc[PREV]);
    advance();
  };

  using I0 = std::integral_constant<int, 0>;
  using I1 = std::integral_constant<int, 1>;
  using I2 = std::integral_constant<int, 2>;
  // Trips of three steps keep the accumulator rotation (k mod 3) compile-time and match the
  // ring's slots: one wait before the trip, one refill after it.  A trip whose three rows are
  // all interior and away from frame edges runs the lean steps, any other trip the general ones.
  int slot = 0;
  uint32_t par = 0u;  // parity of ring pass k / DW_STAGES
#pragma unroll 1
  for (int k = 0; k < nin; k += 3) {
    if (exists(k) || exists(k + 1) || exists(k + 2)) dw_wait(bars + 8 * slot, par);
    const int rs = 3 * slot;
    if (k >= 2 && k + 2 <= nin - 3 && fr >= 1 && fr + 2 <= p.H - 2) {
      step_mid(rs, I0{}, I1{}, I2{});
      step_mid(rs + 1, I1{}, I2{}, I0{});
      step_mid(rs + 2, I2{}, I0{}, I1{});
    } else {
      step_any(k, rs, I0{}, I1{}, I2{});
      if (k + 1 < nin) step_any(k + 1, rs + 1, I1{}, I2{}, I0{});
      if (k + 2 < nin) step_any(k + 2, rs + 2, I2{}, I0{}, I1{});
    }
    // every lane has consumed the slot (its values sit in accumulators): lane 0 may refill it
    __syncwarp();
    if (lane == 0) refill(k + DW_STAGES, slot);
    if (++slot == DW_SLOTS) slot = 0, par ^= 1u;
  }
  if (p.amax_out != nullptr) {
    float m = fmaxf(bf16_lo(amax_bits), bf16_hi(amax_bits));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) atomicMax(reinterpret_cast<unsigned int*>(p.amax_out), __float_as_uint(m));  // m >= 0
  }
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

static int dwconv_glu_impl(const void* u, const void* halo_top, const void* halo_bot, const void* weight, const void* bias,
                           void* out, int64_t rows, int64_t W, int64_t H, int64_t row0, int64_t hid, int dtype,
                           float* amax_out, void* stream) {
  SANA_REQUIRE(u && weight && out, "sana_dwconv_glu: null pointer");
  SANA_REQUIRE(!amax_out || dtype == SANA_BF16, "sana_dwconv_glu_amax: bf16 only");
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
    a.weight = static_cast<const __nv_bfloat16*>(weight);
    a.bias = static_cast<const __nv_bfloat16*>(bias);
    a.out = static_cast<__nv_bfloat16*>(out);
    a.rows = (int)rows, a.W = (int)W, a.H = (int)H, a.hid = (int)hid, a.row0 = row0;
    a.amax_out = amax_out;
    // u as a 4-D tensor {channel, value/gate, x, row}; a box is 64 channels x 2 groups x 4 pixels of one row
    CUtensorMap tmU3, tmU, tmTop, tmBot;
    const uint64_t strides[3] = {(uint64_t)hid * 2, (uint64_t)hid * 4, (uint64_t)W * hid * 4};
    const uint32_t box[4] = {DW_CH, 2, 4, 1};
    const uint64_t dims_u[4] = {(uint64_t)hid, 2, (uint64_t)W, (uint64_t)rows};
    const uint64_t dims_1[4] = {(uint64_t)hid, 2, (uint64_t)W, 1};
    const uint32_t box3[4] = {DW_CH, 2, 4, 3};
    int rc = make_tmap_tiled(&tmU, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, u, dims_u, strides, box, false);
    if (rc) return rc;
    tmU3 = tmU;  // with fewer than three rows the three-row copy is never issued
    if (rows >= 3) {
      rc = make_tmap_tiled(&tmU3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, u, dims_u, strides, box3, false);
      if (rc) return rc;
    }
    tmTop = tmU, tmBot = tmU;
    if (halo_top) {
      rc = make_tmap_tiled(&tmTop, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, halo_top, dims_1, strides, box, false);
      if (rc) return rc;
    }
    if (halo_bot) {
      rc = make_tmap_tiled(&tmBot, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, halo_bot, dims_1, strides, box, false);
      if (rc) return rc;
    }
    const int64_t gx = ceil_div(hid, DW_CH), gy = ceil_div(W, DW_TW);
    // rows per warp: long segments amortise the two halo rows and the warp's set-up; shorten them
    // until the grid covers the device a few times over.
    // (a warp's set-up - 36 weight loads, 9 row fetches - costs about ten rows of work)
    const int64_t slots = (int64_t)sm_count() * DW_CTAS_PER_SM;
    // measured at 1.6B width: 128-256 rows per warp are 17 % faster than 32 as long as at least
    // four waves of CTAs remain
    int seg = 256;
    while (seg > 32 && gx * gy * ceil_div(rows, seg) < 4 * slots) seg >>= 1;
    while (seg > 4 && gx * gy * ceil_div(rows, seg) < 2 * slots) seg >>= 1;
    a.seg_rows = seg;
    const int64_t gz = ceil_div(rows, seg);
    SANA_REQUIRE(gy < 65536 && gz < 65536, "sana_dwconv_glu: grid too large");
    static OncePerDevice attr_once;
    if (attr_once.first_time()) {
      cudaError_t e = cudaFuncSetAttribute(dwconv_glu_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DW_SMEM_BYTES);
      if (e != cudaSuccess) return cuda_status(e, "cudaFuncSetAttribute(dwconv_glu)");
    }
    dwconv_glu_bf16_kernel<<<dim3((unsigned)gx, (unsigned)gy, (unsigned)gz), DW_THREADS, DW_SMEM_BYTES, st>>>(tmU3, tmU, tmTop, tmBot, a);
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

extern "C" int sana_dwconv_glu(const void* u, const void* halo_top, const void* halo_bot, const void* weight,
                               const void* bias, void* out, int64_t rows, int64_t W, int64_t H, int64_t row0,
                               int64_t hid, int dtype, void* stream) {
  return dwconv_glu_impl(u, halo_top, halo_bot, weight, bias, out, rows, W, H, row0, hid, dtype, nullptr, stream);
}

extern "C" int sana_dwconv_glu_amax(const void* u, const void* halo_top, const void* halo_bot, const void* weight,
                                    const void* bias, void* out, int64_t rows, int64_t W, int64_t H, int64_t row0,
                                    int64_t hid, float* amax_out, void* stream) {
  SANA_REQUIRE(amax_out, "sana_dwconv_glu_amax: null pointer");
  return dwconv_glu_impl(u, halo_top, halo_bot, weight, bias, out, rows, W, H, row0, hid, SANA_BF16, amax_out, stream);
}

extern "C" int sana_dwconv_glu_take_device_status(int* status_out) {
  if (!status_out) return fail(SANA_ERR_INVALID, "sana_dwconv_glu_take_device_status: null pointer");
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_dw_status, sizeof(int));
  if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyFromSymbol(g_dw_status)");
  if (v != 0) {
    int zero = 0;
    e = cudaMemcpyToSymbol(g_dw_status, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e, "cudaMemcpyToSymbol(g_dw_status)");
  }
  *status_out = v;
  return SANA_OK;
}
