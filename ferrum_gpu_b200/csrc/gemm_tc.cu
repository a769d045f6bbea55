// Scoring-side quantised product on the 5th-generation tensor cores:
//   Y[m, n] = A[m, k] (f16) . dequant(W)[n, k]^T (fp16), f32 accumulators in tensor memory.
// Replaces qlinear_tiled.wgsl for M >= 128 (ferrum_wgpu/src/shaders/quant/qlinear_tiled.wgsl:L93-L128).
//
// Two kernel bodies share the packed-weight readers and dequantisers of this file:
//   - gemm_ts_main.cuh: the weight rows on the tensor-memory lanes. A producer thread owns one weight row = one
//     lane, dequantises its packed blocks of a 64-k slice and writes them into tensor memory, from where they are
//     the MMA's A operand; the activations (192 rows x 64 f16 per TMA box) are the B operand. f32 / fp16 /
//     residual / SwiGLU results leave through shared memory and bulk tensor stores. Every product but the head.
//   - gemm_tc_main.cuh: the activation rows on the lanes, 256 x 128 tiles, both operands in shared memory (the
//     weight slice dequantised into the swizzled K-major layout TMA produces). The vocabulary head: its epilogue
//     folds a row of logits into (max, sum-exp, target logit, first argmax) in one thread's registers.
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr int STAGES = 3;
constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2; // 32 KB: two 128-row halves
constexpr uint32_t B_BYTES = TC_BN * TC_BK * 2; // 16 KB
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 640; // 20 warps: TMA, MMA, 2 idle, 8 producers, 8 epilogue
constexpr uint32_t TMEM_COLS = 512; // two tiles x two accumulators x 128 columns
// setmaxnreg targets of the three warp classes (4 control, 8 producer, 8 epilogue warps). The pool
// they draw on is what the CTA was launched with (threads x registers per thread as compiled), and
// an increase that does not fit waits forever, so the launch code checks the sum against the compiled
// register count before the first launch.
constexpr int REGS_CTRL = 40, REGS_PROD = 64, REGS_EPI = 152;
constexpr int REGS_NEEDED = 32 * (4 * REGS_CTRL + 8 * REGS_PROD + 8 * REGS_EPI);

// The kernel with the weights on the tensor-memory lanes (gemm_ts_main.cuh)
constexpr uint32_t TS_BX = 192;                   // activation rows per tile: the MMA's N
constexpr int X_STAGES = 6, W_STAGES = 4;
constexpr uint32_t X_BYTES = TS_BX * TC_BK * 2;   // 24 KB: one TMA box
constexpr uint32_t W_COLS = TC_BK / 2;            // tensor-memory columns of one weight stage (two f16 per column)
constexpr uint32_t W_COL0 = 2 * TS_BX;            // after the two accumulator buffers
static_assert(W_COL0 + W_STAGES * W_COLS <= 512, "tensor memory has 512 columns");
constexpr uint32_t STG_OFF = X_STAGES * X_BYTES + 512; // after the rings and the barriers
constexpr uint32_t STG_TILE = 32 * 32 * 4;        // one staged chunk of an epilogue warp (two per warp)
constexpr uint32_t TS_SMEM_BYTES = STG_OFF + 8 * 2 * STG_TILE + 1024 /*alignment slack*/;
constexpr int PSETS = 3;                          // producer sets of four warps
constexpr int TS_THREADS = (4 + 4 * PSETS + 8) * 32;
// setmaxnreg targets: 4 control warps, 4 * PSETS producer warps, 8 epilogue warps; the sum must fit the registers
// the CTA is launched with (checked before the first launch)
constexpr int TS_REGS_PROD = 64, TS_REGS_EPI = 120;
constexpr int TS_REGS_NEEDED = 32 * (4 * REGS_CTRL + 4 * PSETS * TS_REGS_PROD + 8 * TS_REGS_EPI);

// The batched-decode product at f32-class accuracy (gemm_tx_main.cuh)
constexpr int TX_X_STAGES = 8, TX_W_STAGES = 4, TX_PSETS = 2;
constexpr uint32_t TX_CHUNK = 4;                  // K steps (256 k) that tensor memory accumulates before the registers take over
constexpr uint32_t TX_X_BYTES = 128 * TC_BK * 2;  // 16 KB: the xh box over the xl box
constexpr uint32_t TX_Q_OFF = TX_X_BYTES;         // then the tile's packed weights of the step (128 rows of 64 or 32 bytes)
constexpr uint32_t TX_SC_OFF = TX_Q_OFF + 8192;   // then eight f16 scales per row (the step's 256-k chunk)
constexpr uint32_t TX_STAGE_BYTES = TX_SC_OFF + 2048; // 26 KB
constexpr uint32_t TX_ACC_COLS = 128;             // wh.xh (64) | wh.xl + wl.xh (64)
constexpr uint32_t TX_W_COLS = TC_BK;             // 32 columns of wh and 32 of wl per stage
constexpr uint32_t TX_W_COL0 = 2 * TX_ACC_COLS;
static_assert(TX_W_COL0 + TX_W_STAGES * TX_W_COLS <= 512, "tensor memory has 512 columns");
constexpr int TX_THREADS = (4 + 4 * TX_PSETS + 8) * 32;
constexpr uint32_t TX_SMEM_BYTES = TX_X_STAGES * TX_STAGE_BYTES + 512 /*barriers*/ + 4 * TC_BN * 4 /*row scales*/ + 1024 /*alignment slack*/;

enum { ERR_WAIT_EMPTY = 1, ERR_WAIT_FULL = 2, ERR_WAIT_ACC = 3 };

// Both operands are fp16 (f32 accumulation). The block scale is an f16 and a quant has at most 8
// bits, so d * q rounds once to 11 bits; bf16 operands (8 bits) miss the 2e-2 per-logit bound of this
// path by a factor of 1.6 on the 12-layer scoring model, fp16 operands meet it with a 6x margin.
// Activations saturate at the fp16 range instead of overflowing to infinity.
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t f16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t f16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Where a dequantised weight row goes, 16 bytes (eight f16 along K) at a time; chunk c covers k = 8c .. 8c + 7
// of the 64-k slice and the chunks of a row come in ascending order.
//
// Into tensor memory: the row is one lane, the slice 32 columns of two f16 each; the sink gathers the four chunks
// of a 32-k block and writes them with one 16-column store.
// Into the shared-memory ring of the kernel that reads both operands from there: the K-major layout TMA produces,
// 128-byte rows whose 16-byte chunks are XORed with the row number (128B swizzle).
struct SmemSink {
  uint32_t row_smem, sw;
  template <int C>
  __device__ __forceinline__ void put(uint32_t o0, uint32_t o1, uint32_t o2, uint32_t o3) {
    const uint32_t addr = row_smem + ((((uint32_t)C) ^ sw) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o0), "r"(o1), "r"(o2), "r"(o3) : "memory");
  }
};
struct TmemSink {
  uint32_t taddr; // lane base of this warp | first column of the stage
  uint32_t v[16];
  template <int C>
  __device__ __forceinline__ void put(uint32_t o0, uint32_t o1, uint32_t o2, uint32_t o3) {
    v[(C & 3) * 4 + 0] = o0, v[(C & 3) * 4 + 1] = o1, v[(C & 3) * 4 + 2] = o2, v[(C & 3) * 4 + 3] = o3;
    if ((C & 3) == 3) tc::tmem_st_32x16(taddr + (C >> 2) * 16, v);
  }
};

// One 32-element Q4_0 block (4 words, device nibble order) -> chunks C0 .. C0 + 3
template <int C0, class Sink>
__device__ __forceinline__ void dequant_q4_block(const uint4& q, __half d, Sink& sink) {
  const uint32_t dd = (uint32_t)__half_as_ushort(d) * 0x00010001u; // the f16 scale in both halves
  const uint32_t words[4] = {q.x, q.y, q.z, q.w};
  auto one = [&](uint32_t w, uint32_t (&o)[4]) {
    // nibbles p and p+4 of the word are elements 2p and 2p+1. In the low four mantissa bits of 0x6400 a nibble
    // makes the fp16 1024 + nib, four bits higher under 0x5400 it makes 64 + nib: no shift for the odd places
    const uint32_t w8 = w >> 8;
    const uint32_t t0 = (w & 0x000f000fu) | 0x64006400u, t1 = (w & 0x00f000f0u) | 0x54005400u;
    const uint32_t t2 = (w8 & 0x000f000fu) | 0x64006400u, t3 = (w8 & 0x00f000f0u) | 0x54005400u;
    o[0] = f16x2_mul(f16x2_sub(t0, 0x64086408u), dd); // - 1032: exact, (nib - 8); then one rounding
    o[1] = f16x2_mul(f16x2_sub(t1, 0x54805480u), dd); // - 72
    o[2] = f16x2_mul(f16x2_sub(t2, 0x64086408u), dd);
    o[3] = f16x2_mul(f16x2_sub(t3, 0x54805480u), dd);
  };
  uint32_t o[4];
  one(words[0], o), sink.template put<C0>(o[0], o[1], o[2], o[3]);
  one(words[1], o), sink.template put<C0 + 1>(o[0], o[1], o[2], o[3]);
  one(words[2], o), sink.template put<C0 + 2>(o[0], o[1], o[2], o[3]);
  one(words[3], o), sink.template put<C0 + 3>(o[0], o[1], o[2], o[3]);
}

// 16 int8 quants (one uint4 = half a Q8_0 block) -> chunks C0, C0 + 1. A byte b = q + 128 under the exponent byte
// 0x64 is the fp16 1024 + b; minus 1152 leaves q exactly, and one half2 multiply by the block's f16 scale (`dd`: in
// both halves) rounds d * q to fp16 once - the same bits as the f32 product (exact: 19 bits) converted to fp16.
template <int C0, class Sink>
__device__ __forceinline__ void dequant_q8_half(const uint4& q, uint32_t dd, Sink& sink) {
  auto one = [&](uint32_t wa, uint32_t wb, uint32_t (&o)[4]) {
    const uint32_t ua = wa ^ 0x80808080u, ub = wb ^ 0x80808080u;
    o[0] = f16x2_mul(f16x2_sub(__byte_perm(ua, 0x64646464u, 0x5140), 0x64806480u), dd);
    o[1] = f16x2_mul(f16x2_sub(__byte_perm(ua, 0x64646464u, 0x5342), 0x64806480u), dd);
    o[2] = f16x2_mul(f16x2_sub(__byte_perm(ub, 0x64646464u, 0x5140), 0x64806480u), dd);
    o[3] = f16x2_mul(f16x2_sub(__byte_perm(ub, 0x64646464u, 0x5342), 0x64806480u), dd);
  };
  uint32_t o[4];
  one(q.x, q.y, o), sink.template put<C0>(o[0], o[1], o[2], o[3]);
  one(q.z, q.w, o), sink.template put<C0 + 1>(o[0], o[1], o[2], o[3]);
}

// One 32-element MXFP4 block (4 words, element order) -> chunks C0 .. C0 + 3: E2M1 value times the power-of-two
// scale in f32 (the scale itself need not be an fp16 value), saturated to fp16
template <int C0, class Sink>
__device__ __forceinline__ void dequant_mxfp4_block(const uint4& q, float d, Sink& sink) {
  auto one = [&](uint32_t w, uint32_t (&o)[4]) {
    uint32_t h[4];
    e2m1x8_to_f16x2(w, h);
#pragma unroll
    for (int p = 0; p < 4; p++) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[p]));
      o[p] = pack_f16(f.x * d, f.y * d);
    }
  };
  uint32_t o[4];
  one(q.x, o), sink.template put<C0>(o[0], o[1], o[2], o[3]);
  one(q.y, o), sink.template put<C0 + 1>(o[0], o[1], o[2], o[3]);
  one(q.z, o), sink.template put<C0 + 2>(o[0], o[1], o[2], o[3]);
  one(q.w, o), sink.template put<C0 + 3>(o[0], o[1], o[2], o[3]);
}

// 16 FP8 codes (half a block) -> chunks C0, C0 + 1: code -> fp16 exactly, times the f16 scale, one rounding
template <int KIND, int C0, class Sink>
__device__ __forceinline__ void dequant_fp8_half(const uint4& q, __half d, Sink& sink) {
  const uint32_t dd = (uint32_t)__half_as_ushort(d) * 0x00010001u;
  auto one = [&](uint32_t wa, uint32_t wb, uint32_t (&o)[4]) {
    o[0] = f16x2_mul(fp8x2_to_f16x2<KIND>(wa), dd);
    o[1] = f16x2_mul(fp8x2_to_f16x2<KIND>(wa >> 16), dd);
    o[2] = f16x2_mul(fp8x2_to_f16x2<KIND>(wb), dd);
    o[3] = f16x2_mul(fp8x2_to_f16x2<KIND>(wb >> 16), dd);
  };
  uint32_t o[4];
  one(q.x, q.y, o), sink.template put<C0>(o[0], o[1], o[2], o[3]);
  one(q.z, q.w, o), sink.template put<C0 + 1>(o[0], o[1], o[2], o[3]);
}

__device__ __forceinline__ float gelu_f(float x) {
  const float K = 0.7978846f;
  return 0.5f * x * (1.0f + tanhf(K * (x + 0.044715f * x * x * x)));
}

template <int KIND>
struct RowRegs; // packed data of one weight row for one K slice
template <>
struct RowRegs<FC_Q4_0> {
  uint4 q[2];
  uint32_t sc;
};
template <>
struct RowRegs<FC_Q8_0> {
  uint4 q[4];
  uint32_t sc;
};
template <>
struct RowRegs<FC_Q2_K> {
  uint4 q[1];   // 64 two-bit levels: word j is sub-block j (an array so the other kinds' branches still parse)
  uint32_t sc;  // the four sub-blocks' scale / min bytes
  uint32_t dd;  // d | dmin << 16 (f16 bits) of the super-block
};
template <>
struct RowRegs<FC_MXFP4> {
  uint4 q[2];
  uint32_t sc;
};
template <>
struct RowRegs<FC_FP8_E4M3> {
  uint4 q[4];
  uint32_t sc;
};
template <>
struct RowRegs<FC_FP8_E5M2> {
  uint4 q[4];
  uint32_t sc;
};
template <>
struct RowRegs<FC_F32> {
  uint4 q[16];
};
template <>
struct RowRegs<FC_F16> {
  uint4 q[8];
};

template <int KIND>
__device__ __forceinline__ void load_row(RowRegs<KIND>& r, const QMat& w, uint32_t row, uint32_t it, bool valid) {
  if (KIND == FC_Q2_K) { // a 64-k slice is a quarter of a super-block; rows past the end decode to zero
    RowRegs<FC_Q2_K>& rr = (RowRegs<FC_Q2_K>&)r;
    const uint32_t* rec =
        reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(w.sc) + ((size_t)row * (w.k / QK_K) + (it >> 2)) * 20);
    rr.q[0] = valid ? __ldg(reinterpret_cast<const uint4*>(w.qs + (size_t)row * (w.k / 4) + (size_t)it * 16)) : make_uint4(0, 0, 0, 0);
    rr.sc = valid ? __ldg(rec + (it & 3)) : 0u;
    rr.dd = valid ? __ldg(rec + 4) : 0u;
  } else if (kind_nibble_blocks(KIND)) { // (rows past the end decode to zero: nibble 8 of Q4_0, code 0 of MXFP4)
    const uint32_t zero = KIND == FC_Q4_0 ? 0x88888888u : 0u;
    const uint4* p = reinterpret_cast<const uint4*>(w.qs + (size_t)row * (w.k / 2) + (size_t)it * 32);
    r.q[0] = valid ? __ldg(p) : make_uint4(zero, zero, zero, zero);
    r.q[1] = valid ? __ldg(p + 1) : make_uint4(zero, zero, zero, zero);
    *reinterpret_cast<uint32_t*>(&((RowRegs<FC_Q4_0>&)r).sc) =
        valid ? __ldg(reinterpret_cast<const uint32_t*>(w.sc + (size_t)row * (w.k / QK) + (size_t)it * 2)) : 0u;
  } else if (kind_byte_blocks(KIND)) { // (the three records have one layout)
    const uint4* p = reinterpret_cast<const uint4*>(w.qs + (size_t)row * w.k + (size_t)it * 64);
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = valid ? __ldg(p + i) : make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint32_t*>(&((RowRegs<FC_Q8_0>&)r).sc) =
        valid ? __ldg(reinterpret_cast<const uint32_t*>(w.sc + (size_t)row * (w.k / QK) + (size_t)it * 2)) : 0u;
  } else if (KIND == FC_F16) {
    const uint4* p = reinterpret_cast<const uint4*>(w.qs + ((size_t)row * w.k + (size_t)it * 64) * 2);
#pragma unroll
    for (int i = 0; i < 8; i++) r.q[i] = valid ? __ldg(p + i) : make_uint4(0, 0, 0, 0);
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(w.qs + ((size_t)row * w.k + (size_t)it * 64) * 4);
#pragma unroll
    for (int i = 0; i < 16; i++) r.q[i] = valid ? __ldg(p + i) : make_uint4(0, 0, 0, 0);
  }
}

template <int KIND, class Sink>
__device__ __forceinline__ void emit_row(const RowRegs<KIND>& r, Sink& sink) {
  if (KIND == FC_Q4_0) {
    const RowRegs<FC_Q4_0>& rr = (const RowRegs<FC_Q4_0>&)r;
    const __half d0 = __ushort_as_half((unsigned short)(rr.sc & 0xffff)), d1 = __ushort_as_half((unsigned short)(rr.sc >> 16));
    dequant_q4_block<0>(rr.q[0], d0, sink);
    dequant_q4_block<4>(rr.q[1], d1, sink);
  } else if (KIND == FC_Q8_0) {
    const RowRegs<FC_Q8_0>& rr = (const RowRegs<FC_Q8_0>&)r;
    const uint32_t d0 = (rr.sc & 0xffffu) * 0x00010001u, d1 = (rr.sc >> 16) * 0x00010001u; // the f16 scale in both halves
    dequant_q8_half<0>(rr.q[0], d0, sink);
    dequant_q8_half<2>(rr.q[1], d0, sink);
    dequant_q8_half<4>(rr.q[2], d1, sink);
    dequant_q8_half<6>(rr.q[3], d1, sink);
  } else if (KIND == FC_Q2_K) { // (d * sc) * q - dmin * m in f32, one rounding to fp16
    const RowRegs<FC_Q2_K>& rr = (const RowRegs<FC_Q2_K>&)r;
    const float d = __half2float(__ushort_as_half((unsigned short)(rr.dd & 0xffffu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(rr.dd >> 16)));
    auto one = [&](uint32_t word, uint32_t scb, int h, uint32_t (&o)[4]) {
      const float dl = d * (float)(scb & 15u), ml = dmin * (float)(scb >> 4);
      const uint32_t b = word >> (16 * h);
#pragma unroll
      for (int p = 0; p < 4; p++)
        o[p] = pack_f16(fmaf(dl, (float)((b >> (4 * p)) & 3u), -ml), fmaf(dl, (float)((b >> (4 * p + 2)) & 3u), -ml));
    };
    uint32_t o[4];
    one(rr.q[0].x, rr.sc & 0xffu, 0, o), sink.template put<0>(o[0], o[1], o[2], o[3]);
    one(rr.q[0].x, rr.sc & 0xffu, 1, o), sink.template put<1>(o[0], o[1], o[2], o[3]);
    one(rr.q[0].y, (rr.sc >> 8) & 0xffu, 0, o), sink.template put<2>(o[0], o[1], o[2], o[3]);
    one(rr.q[0].y, (rr.sc >> 8) & 0xffu, 1, o), sink.template put<3>(o[0], o[1], o[2], o[3]);
    one(rr.q[0].z, (rr.sc >> 16) & 0xffu, 0, o), sink.template put<4>(o[0], o[1], o[2], o[3]);
    one(rr.q[0].z, (rr.sc >> 16) & 0xffu, 1, o), sink.template put<5>(o[0], o[1], o[2], o[3]);
    one(rr.q[0].w, rr.sc >> 24, 0, o), sink.template put<6>(o[0], o[1], o[2], o[3]);
    one(rr.q[0].w, rr.sc >> 24, 1, o), sink.template put<7>(o[0], o[1], o[2], o[3]);
  } else if (KIND == FC_MXFP4) {
    const RowRegs<FC_Q4_0>& rr = (const RowRegs<FC_Q4_0>&)r;
    dequant_mxfp4_block<0>(rr.q[0], __uint_as_float(rr.sc << 16), sink);
    dequant_mxfp4_block<4>(rr.q[1], __uint_as_float(rr.sc & 0xffff0000u), sink);
  } else if (kind_is_fp8(KIND)) {
    const RowRegs<FC_Q8_0>& rr = (const RowRegs<FC_Q8_0>&)r;
    const __half d0 = __ushort_as_half((unsigned short)(rr.sc & 0xffff)), d1 = __ushort_as_half((unsigned short)(rr.sc >> 16));
    dequant_fp8_half<KIND, 0>(rr.q[0], d0, sink);
    dequant_fp8_half<KIND, 2>(rr.q[1], d0, sink);
    dequant_fp8_half<KIND, 4>(rr.q[2], d1, sink);
    dequant_fp8_half<KIND, 6>(rr.q[3], d1, sink);
  } else if (KIND == FC_F16) { // stored values are the operand
    const RowRegs<FC_F16>& rr = (const RowRegs<FC_F16>&)r;
    sink.template put<0>(rr.q[0].x, rr.q[0].y, rr.q[0].z, rr.q[0].w);
    sink.template put<1>(rr.q[1].x, rr.q[1].y, rr.q[1].z, rr.q[1].w);
    sink.template put<2>(rr.q[2].x, rr.q[2].y, rr.q[2].z, rr.q[2].w);
    sink.template put<3>(rr.q[3].x, rr.q[3].y, rr.q[3].z, rr.q[3].w);
    sink.template put<4>(rr.q[4].x, rr.q[4].y, rr.q[4].z, rr.q[4].w);
    sink.template put<5>(rr.q[5].x, rr.q[5].y, rr.q[5].z, rr.q[5].w);
    sink.template put<6>(rr.q[6].x, rr.q[6].y, rr.q[6].z, rr.q[6].w);
    sink.template put<7>(rr.q[7].x, rr.q[7].y, rr.q[7].z, rr.q[7].w);
  } else {
    const RowRegs<FC_F32>& rr = (const RowRegs<FC_F32>&)r;
    auto one = [&](const uint4& a, const uint4& b, uint32_t (&o)[4]) {
      o[0] = pack_f16(__uint_as_float(a.x), __uint_as_float(a.y));
      o[1] = pack_f16(__uint_as_float(a.z), __uint_as_float(a.w));
      o[2] = pack_f16(__uint_as_float(b.x), __uint_as_float(b.y));
      o[3] = pack_f16(__uint_as_float(b.z), __uint_as_float(b.w));
    };
    uint32_t o[4];
    one(rr.q[0], rr.q[1], o), sink.template put<0>(o[0], o[1], o[2], o[3]);
    one(rr.q[2], rr.q[3], o), sink.template put<1>(o[0], o[1], o[2], o[3]);
    one(rr.q[4], rr.q[5], o), sink.template put<2>(o[0], o[1], o[2], o[3]);
    one(rr.q[6], rr.q[7], o), sink.template put<3>(o[0], o[1], o[2], o[3]);
    one(rr.q[8], rr.q[9], o), sink.template put<4>(o[0], o[1], o[2], o[3]);
    one(rr.q[10], rr.q[11], o), sink.template put<5>(o[0], o[1], o[2], o[3]);
    one(rr.q[12], rr.q[13], o), sink.template put<6>(o[0], o[1], o[2], o[3]);
    one(rr.q[14], rr.q[15], o), sink.template put<7>(o[0], o[1], o[2], o[3]);
  }
}

// ---- epilogues -------------------------------------------------------------------------------------

__device__ __forceinline__ float ex2f_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct LseState {
  float mx = -INFINITY, se = 0.0f, tl = -INFINITY;
  int first = 0;
};
// Folds 32 consecutive logits of one row (columns [col0, col0 + 32) of this rank's vocabulary slice)
// into the row's running (max, sum of exp, target logit, first argmax).
__device__ __forceinline__ void epilogue_lse(const TcArgs& a, LseState& s, uint32_t col0, int target, uint32_t* acc) {
  constexpr float LOG2E = 1.4426950408889634f;
  if (col0 >= a.n) return;
  if (col0 + 32 > a.n) { // ragged last chunk: columns past the vocabulary never win and add nothing
#pragma unroll
    for (int j = 0; j < 32; j++)
      if (col0 + j >= a.n) acc[j] = 0xff800000u;
  }
  float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    m4[0] = fmaxf(m4[0], __uint_as_float(acc[j]));
    m4[1] = fmaxf(m4[1], __uint_as_float(acc[j + 1]));
    m4[2] = fmaxf(m4[2], __uint_as_float(acc[j + 2]));
    m4[3] = fmaxf(m4[3], __uint_as_float(acc[j + 3]));
  }
  const float cm = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
  if (cm > s.mx) { // strictly greater: an earlier chunk keeps a tied maximum
    s.se *= ex2f_approx((s.mx - cm) * LOG2E);
    s.mx = cm;
    int f = 31;
#pragma unroll
    for (int j = 30; j >= 0; j--)
      if (__uint_as_float(acc[j]) == cm) f = j; // descending: the first occurrence is written last
    s.first = (int)(a.v0 + col0) + f;
  }
  const int tj = target - (int)(a.v0 + col0);
  if (tj >= 0 && tj < 32) {
#pragma unroll
    for (int j = 0; j < 32; j++)
      if (j == tj) s.tl = __uint_as_float(acc[j]);
  }
  const float msc = s.mx * LOG2E;
  float e4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    e4[0] += ex2f_approx(fmaf(__uint_as_float(acc[j]), LOG2E, -msc));
    e4[1] += ex2f_approx(fmaf(__uint_as_float(acc[j + 1]), LOG2E, -msc));
    e4[2] += ex2f_approx(fmaf(__uint_as_float(acc[j + 2]), LOG2E, -msc));
    e4[3] += ex2f_approx(fmaf(__uint_as_float(acc[j + 3]), LOG2E, -msc));
  }
  s.se += (e4[0] + e4[1]) + (e4[2] + e4[3]);
}

#include "gemm_tc_main.cuh"
#include "gemm_ts_main.cuh"
#include "gemm_tx_main.cuh"

// cuTensorMapEncodeTiled through the runtime's driver entry point: the library carries no link
// dependency on libcuda, so it still loads (and exports its symbols) on a machine without a GPU.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

template <int KIND, int EPI>
int launch_tc(FcDevice* dev, const CUtensorMap& tmap, const QMat& w, const TcArgs& a, dim3 grid) {
  auto kern = qgemm_tc_kernel<KIND, EPI>;
  static OncePerDevice attr; // one per instantiation
  if (attr.first(dev->ordinal)) {
    attr.again(dev->ordinal); // (until the checks below have passed)
    cudaFuncAttributes fa;
    FC_CUDA(dev, cudaFuncGetAttributes(&fa, kern));
    if (fa.numRegs * THREADS < REGS_NEEDED)
      return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensor-core product was compiled with %d registers per thread; its register "
                     "rebalancing needs %d", fa.numRegs, (REGS_NEEDED + THREADS - 1) / THREADS);
    FC_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    attr.first(dev->ordinal);
  }
  FC_LAUNCH(dev, "qgemm_tc_lse", kern<<<grid, THREADS, SMEM_BYTES, dev->stream>>>(tmap, w, a));
  return FC_OK;
}

template <int KIND, int EPI>
int launch_ts(FcDevice* dev, const CUtensorMap& tmap, const QMat& w, TcArgs a, dim3 grid) {
  // The output as a TMA tensor of 32 x 32 boxes (16 columns wide for SwiGLU's halved output), when its base and
  // row pitch are whole 16 bytes; otherwise the epilogue stores from registers.
  CUtensorMap tmap_o = tmap;
  {
    const bool f32 = EPI == EPI_F32 || EPI == EPI_RESID;
    void* out = f32 ? (void*)a.out_f32 : (void*)a.out_f16;
    const uint64_t pitch = (uint64_t)a.ldo * (f32 ? 4 : 2);
    const uint64_t cols = EPI == EPI_SWIGLU ? w.n / 2 : w.n;
    if (out && pitch % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && cols > 0) {
      const cuuint64_t dims[2] = {cols, a.m};
      const cuuint64_t strides[1] = {pitch};
      const cuuint32_t box[2] = {EPI == EPI_SWIGLU ? 16u : 32u, 32u};
      const cuuint32_t estr[2] = {1, 1};
      CUresult cr = encode_fn()(&tmap_o, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, out, dims, strides,
                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled (output) failed with %d", (int)cr);
      a.out_tma = 1;
    }
  }
  auto kern = qgemm_ts_kernel<KIND, EPI>;
  static OncePerDevice attr; // one per instantiation
  if (attr.first(dev->ordinal)) {
    attr.again(dev->ordinal); // (until the checks below have passed)
    cudaFuncAttributes fa;
    FC_CUDA(dev, cudaFuncGetAttributes(&fa, kern));
    if (fa.numRegs * TS_THREADS < TS_REGS_NEEDED)
      return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensor-core product was compiled with %d registers per thread; its register "
                     "rebalancing needs %d", fa.numRegs, (TS_REGS_NEEDED + TS_THREADS - 1) / TS_THREADS);
    FC_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TS_SMEM_BYTES));
    attr.first(dev->ordinal);
  }
  static const char* const names[] = {"qgemm_tc_f32", "qgemm_tc_f16", "qgemm_tc_resid", "qgemm_tc_swiglu"};
  FC_LAUNCH(dev, names[EPI], kern<<<grid, TS_THREADS, TS_SMEM_BYTES, dev->stream>>>(tmap, tmap_o, w, a));
  return FC_OK;
}

template <int KIND>
int pick_epi_ts(FcDevice* dev, const CUtensorMap& tmap, const QMat& w, const TcArgs& a, int epi, dim3 grid) {
  switch (epi) {
    case EPI_F32: return launch_ts<KIND, EPI_F32>(dev, tmap, w, a, grid);
    case EPI_F16: return launch_ts<KIND, EPI_F16>(dev, tmap, w, a, grid);
    case EPI_RESID: return launch_ts<KIND, EPI_RESID>(dev, tmap, w, a, grid);
    case EPI_SWIGLU: return launch_ts<KIND, EPI_SWIGLU>(dev, tmap, w, a, grid);
  }
  return fc_fail(dev, FC_ERR_ARG, "unknown epilogue %d", epi);
}

template <int KIND>
int pick_epi(FcDevice* dev, const CUtensorMap& tmap, const QMat& w, const TcArgs& a, int epi, dim3 grid) {
  if (epi == EPI_LSE) return launch_tc<KIND, EPI_LSE>(dev, tmap, w, a, grid);
  return fc_fail(dev, FC_ERR_ARG, "unknown epilogue %d", epi);
}

template <int KIND>
int launch_tx(FcDevice* dev, const CUtensorMap& txh, const CUtensorMap& txl, const CUtensorMap& tq, const CUtensorMap& tsc,
              const TxArgs& a, dim3 grid) {
  auto kern = qgemm_tx_kernel<KIND>;
  static OncePerDevice attr;
  if (attr.first(dev->ordinal)) {
    FC_CUDA(dev, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TX_SMEM_BYTES));
  }
  FC_LAUNCH(dev, "qgemm_tx", kern<<<grid, TX_THREADS, TX_SMEM_BYTES, dev->stream>>>(txh, txl, tq, tsc, a));
  return FC_OK;
}

} // namespace

// Whether the product of `m` rows of x takes the exact-class tcgen05 kernel: Q8_0 / Q4_0, 9..64 rows (up to eight
// rows the mma.sync kernel with x in registers streams the weights faster: 50 against 71 us on K 1024 x N 151936),
// whole 256-wide rows of at least 8 K steps, and an output long enough without a split of K: 128-row tiles for half
// of the SMs, or for a quarter of them when more than 32 rows make the mma.sync product slow (K 4096 x N 5120 at 64
// rows: 37 against 41 + 9 us for the product and its split-K reduce) - unless the caller would fold that reduce
// into its next launch (`deferring`), which makes the two even there.
bool qgemm_tx_takes(const FcDevice* dev, const QMat& w, uint32_t m, bool deferring) {
  if (w.kind != FC_Q8_0 && w.kind != FC_Q4_0) return false;
  if (m <= 8 || m > 64 || w.k % 256 || w.k < 512) return false;
  if ((reinterpret_cast<uintptr_t>(w.qs) | reinterpret_cast<uintptr_t>(w.sc)) & 15) return false;
  const uint32_t sms = (uint32_t)dev->prop.multiProcessorCount;
  return (w.n + TC_BN - 1) / TC_BN >= ((m > 32 && !deferring) ? sms / 4 : sms / 2);
}

// y[m][n] = epilogue(x . W^T), x given as its two fp16 terms xh, xl: [mp][k] each, rows m..mp-1 zero.
int k_qgemm_tx(FcDevice* dev, const QMat& w, const __half* xh, const __half* xl, uint32_t mp, uint32_t m, float* y,
               const Epilogue& ep) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap maps[2];
  const __half* src[2] = {xh, xl};
  for (int i = 0; i < 2; i++) {
    if (reinterpret_cast<uintptr_t>(src[i]) & 15) return fc_fail(dev, FC_ERR_ARG, "the split terms of x must be 16-byte aligned");
    const cuuint64_t dims[2] = {w.k, mp};
    const cuuint64_t strides[1] = {(cuuint64_t)w.k * 2};
    const cuuint32_t box[2] = {TC_BK, mp}; // mp = 16, 32 or 64 rows (rows m .. mp - 1 of the buffers are zero)
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&maps[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)src[i], dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled (x terms) failed with %d", (int)cr);
  }
  // the packed weights as bytes, [n][row bytes], in boxes of 128 rows by one K step; the scales, [n][k / 32] f16, in
  // boxes of 128 rows by eight (rows past n read as zeros: scale 0)
  const bool q8 = w.kind == FC_Q8_0;
  const uint32_t row_bytes = q8 ? w.k : w.k / 2, step_bytes = q8 ? 64 : 32;
  CUtensorMap tq, tsc;
  {
    const cuuint64_t dims[2] = {row_bytes, w.n};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {step_bytes, TC_BN};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w.qs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      q8 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled (packed weights) failed with %d", (int)cr);
    const cuuint64_t sdims[2] = {(cuuint64_t)(w.k / QK) * 2, w.n};
    const cuuint64_t sstrides[1] = {(cuuint64_t)(w.k / QK) * 2};
    const cuuint32_t sbox[2] = {16, TC_BN};
    cr = enc(&tsc, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)w.sc, sdims, sstrides, sbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled (scales) failed with %d", (int)cr);
  }
  TxArgs a;
  if (mp != 16 && mp != 32 && mp != 64) return fc_fail(dev, FC_ERR_ARG, "the split terms of x come in blocks of 16, 32 or 64 rows, not %u", mp);
  a.mp = mp;
  a.m = m, a.n = w.n, a.k = w.k, a.y = y, a.bias = ep.bias, a.resid = ep.resid, a.act = ep.act, a.err_flag = dev->d_flag;
  const uint32_t tiles = (w.n + TC_BN - 1) / TC_BN, sms = (uint32_t)dev->prop.multiProcessorCount;
  dim3 grid(tiles < sms ? tiles : sms);
  if (q8) return launch_tx<FC_Q8_0>(dev, maps[0], maps[1], tq, tsc, a, grid);
  return launch_tx<FC_Q4_0>(dev, maps[0], maps[1], tq, tsc, a, grid);
}

int k_qgemm_tc_f16(FcDevice* dev, const QMat& w, const __half* a_dev, int epi, TcArgs args) {
  if (args.m == 0) return FC_OK;
  args.n = w.n;
  args.k = w.k;
  args.err_flag = dev->d_flag;
  if (w.k % TC_BK) return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensor-core product needs k %% 64 == 0, not %u", w.k);
  if ((epi == EPI_F16 || epi == EPI_SWIGLU) && (w.n % 8 || args.ldo % 8))
    return fc_fail(dev, FC_ERR_UNSUPPORTED, "a f16 result needs n %% 8 == 0, not %u", w.n);
  if (epi < EPI_F32 || epi > EPI_LSE) return fc_fail(dev, FC_ERR_ARG, "unknown epilogue %d", epi);
  if ((reinterpret_cast<uintptr_t>(a_dev) & 15) != 0) return fc_fail(dev, FC_ERR_ARG, "the A operand must be 16-byte aligned");
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  // The log-sum-exp head keeps the activation rows on the tensor-memory lanes (a thread folds one row's logits in
  // registers); every other epilogue runs the kernel with the weight rows there.
  const bool on_lanes = epi != EPI_LSE;
  const uint32_t box_rows = on_lanes ? TS_BX : TC_BM;
  CUtensorMap tmap;
  const cuuint64_t dims[2] = {w.k, args.m};
  const cuuint64_t strides[1] = {(cuuint64_t)w.k * 2};
  const cuuint32_t box[2] = {TC_BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)a_dev, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled failed with %d", (int)cr);
  const uint64_t tiles = (uint64_t)((w.n + TC_BN - 1) / TC_BN) * ((args.m + box_rows - 1) / box_rows);
  if (tiles > 0x7fffffffull) return fc_fail(dev, FC_ERR_UNSUPPORTED, "%u rows exceed one launch of the tensor-core product", args.m);
  const uint32_t sms = (uint32_t)dev->prop.multiProcessorCount;
  dim3 grid((unsigned)(tiles < sms ? tiles : sms)); // persistent: one CTA per SM walks the tiles
  if (on_lanes) {
    if (w.kind == FC_Q4_0) return pick_epi_ts<FC_Q4_0>(dev, tmap, w, args, epi, grid);
    if (w.kind == FC_Q8_0) return pick_epi_ts<FC_Q8_0>(dev, tmap, w, args, epi, grid);
    if (w.kind == FC_F16) return pick_epi_ts<FC_F16>(dev, tmap, w, args, epi, grid);
    if (w.kind == FC_FP8_E4M3) return pick_epi_ts<FC_FP8_E4M3>(dev, tmap, w, args, epi, grid);
    if (w.kind == FC_FP8_E5M2) return pick_epi_ts<FC_FP8_E5M2>(dev, tmap, w, args, epi, grid);
    if (w.kind == FC_MXFP4) return pick_epi_ts<FC_MXFP4>(dev, tmap, w, args, epi, grid);
    if (w.kind == FC_Q2_K) return pick_epi_ts<FC_Q2_K>(dev, tmap, w, args, epi, grid);
    return pick_epi_ts<FC_F32>(dev, tmap, w, args, epi, grid);
  }
  if (w.kind == FC_Q4_0) return pick_epi<FC_Q4_0>(dev, tmap, w, args, epi, grid);
  if (w.kind == FC_Q8_0) return pick_epi<FC_Q8_0>(dev, tmap, w, args, epi, grid);
  if (w.kind == FC_F16) return pick_epi<FC_F16>(dev, tmap, w, args, epi, grid);
  if (w.kind == FC_FP8_E4M3) return pick_epi<FC_FP8_E4M3>(dev, tmap, w, args, epi, grid);
  if (w.kind == FC_FP8_E5M2) return pick_epi<FC_FP8_E5M2>(dev, tmap, w, args, epi, grid);
  if (w.kind == FC_MXFP4) return pick_epi<FC_MXFP4>(dev, tmap, w, args, epi, grid);
  if (w.kind == FC_Q2_K) return pick_epi<FC_Q2_K>(dev, tmap, w, args, epi, grid);
  return pick_epi<FC_F32>(dev, tmap, w, args, epi, grid);
}

int tc_check_errors(FcDevice* dev) {
  int flag = 0;
  FC_CUDA(dev, cudaMemcpyAsync(&flag, dev->d_flag, sizeof(int), cudaMemcpyDeviceToHost, dev->stream));
  FC_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (flag != 0) {
    cudaMemsetAsync(dev->d_flag, 0, sizeof(int), dev->stream);
    return fc_fail(dev, FC_ERR_TIMEOUT, "a tensor-core kernel gave up a bounded wait (stage %d)", flag);
  }
  return FC_OK;
}
