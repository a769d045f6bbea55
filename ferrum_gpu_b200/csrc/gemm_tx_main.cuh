// The third kernel body of gemm_tc.cu (included there, inside its anonymous namespace): the batched-decode product
// of 2..64 rows of x at f32-class accuracy on tcgen05, for outputs long enough to fill the device without a split
// of K (vocabulary heads, wide feed-forward layers).
//
//   y[j, n] = sum_k x[j, k] * d[n, k / 32] * q[n, k]            j < m <= 64, tiles of 128 weight rows
//
// Both factors are taken apart into two fp16 terms whose products are exact in the f32 accumulator:
//   x = xh + xl            (22 significant bits; the caller's split buffers, as for the mma.sync product)
//   d * q = wh + wl        (d is an f16 and |q| < 2^8: at most 19 bits, so two fp16 terms hold the product exactly)
//   y = (wh + wl) . xh + (wh + wl) . xl                         (all four cross terms)
// A producer thread owns one weight row (one tensor-memory lane): per 64-k slice it reads the row's packed bytes
// and scales from the stage TMA filled (a thread reading its own row from global memory costs the L1 a tag lookup
// per thread: the kernel was bound by exactly that), forms wh = fp16(d * q) and wl = d * q - wh (one fused
// multiply-add, exact) in half2 arithmetic and writes 32 columns of each into tensor memory. So that wl keeps
// its bits however small the scales are, the row's 256-k chunk is first multiplied by the power of two that brings
// the largest of its eight scales to [2^7, 2^8); the epilogue divides it out chunk by chunk.
// (For at most 32 or 16 rows of x the boxes, the tile and the MMAs' N shrink with them: 2 x 32 or 2 x 16 rows.)
// The B operand of a K step is one shared-memory tile of 128 rows: rows 0..63 the xh slice, rows 64..127 the xl
// slice (two TMA boxes). Two MMAs per 16 k, both against all 128 rows into the same 128 accumulator columns:
// A = wh, then A = wl. Tensor memory: two accumulator buffers of 128 columns, four weight stages of 32 + 32.
//
// The tensor cores' f32 accumulation is not the round-to-nearest chain the exact path is held to: over a whole row
// of 4096 k it was measured ten times further from exact arithmetic than the mma.sync product (7e-7 of sum |x||w|
// against 4e-8). So tensor memory only ever accumulates TX_CHUNK K steps (256 k): the MMA issuer alternates the two
// accumulator buffers chunk by chunk, and the epilogue warps add every finished chunk into f32 registers (a thread
// holds one output column for 32 rows of x) while the next chunk is being multiplied.
//
//   warp 0        TMA: the xh and xl boxes, the packed weights and the chunk's scales of a K step into an 8-deep ring
//   warp 1        tensor-memory owner and MMA issuer
//   warps 4-11    weight producers in two sets of four warps (even and odd K steps)
//   warps 12-19   epilogue: warp w reads lane quadrant w % 4, rows of x [32 (w - 12) / 4, + 32)
//
// Barriers: x_full[s] (TMA bytes), w_full[t] (4 producer warps), x_empty[s] (the MMA commit of the step: frees
// the ring stage and, four steps later, the weight stage), acc_full / acc_empty per 256-k chunk. Every wait is
// bounded and polls the CTA-wide abort word.

// Two fp16 terms of a weight row into tensor memory: `hi` and `lo` stage columns of this warp's lanes.
struct DualTmemSink {
  uint32_t taddr_hi, taddr_lo;
  uint32_t vh[8], vl[8]; // two chunks (16 k) of each term, then one 8-column store each
  template <int C>
  __device__ __forceinline__ void put(const uint32_t (&h)[4], const uint32_t (&l)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) vh[(C & 1) * 4 + i] = h[i], vl[(C & 1) * 4 + i] = l[i];
    if ((C & 1) == 1) {
      tc::tmem_st_32x8(taddr_hi + (C >> 1) * 8, vh);
      tc::tmem_st_32x8(taddr_lo + (C >> 1) * 8, vl);
    }
  }
};
// q (two small integers, exact in fp16) times d (the block's normalised scale in both halves) -> the pair's hi word,
// the product rounded to fp16, and lo word, what the rounding left: one fused multiply-add, exact because the product
// has at most 19 significant bits.
__device__ __forceinline__ void split_pair(uint32_t q2, uint32_t d2, uint32_t& hi, uint32_t& lo) {
  hi = f16x2_mul(q2, d2);
  asm("{\n.reg .b32 n;\nneg.f16x2 n, %3;\nfma.rn.f16x2 %0, %1, %2, n;\n}" : "=r"(lo) : "r"(q2), "r"(d2), "r"(hi));
}
// the block's f16 scale times the chunk's power of two, as an fp16 in both halves (exact: the power of two brought
// the chunk's largest scale to [2^7, 2^8); a scale more than 2^-21 of that may lose low bits to the subnormal range)
__device__ __forceinline__ uint32_t scale_x2(uint32_t sc_bits, float mul) {
  const float d = __half2float(__ushort_as_half((unsigned short)sc_bits)) * mul;
  return (uint32_t)__half_as_ushort(__float2half_rn(d)) * 0x00010001u;
}
template <int KIND>
__device__ __forceinline__ void emit_row_hilo(const RowRegs<KIND>& r, float mul, DualTmemSink& sink) {
  if (KIND == FC_Q8_0) {
    const RowRegs<FC_Q8_0>& rr = (const RowRegs<FC_Q8_0>&)r;
    const uint32_t d0 = scale_x2(rr.sc & 0xffffu, mul), d1 = scale_x2(rr.sc >> 16, mul);
    auto chunk = [&](uint32_t wa, uint32_t wb, uint32_t d, uint32_t (&h)[4], uint32_t (&l)[4]) { // 8 int8 quants
      // a byte b = q + 128 under the exponent byte 0x64 is the fp16 1024 + b; minus 1152 leaves q, exactly
      const uint32_t ua = wa ^ 0x80808080u, ub = wb ^ 0x80808080u;
      split_pair(f16x2_sub(__byte_perm(ua, 0x64646464u, 0x5140), 0x64806480u), d, h[0], l[0]);
      split_pair(f16x2_sub(__byte_perm(ua, 0x64646464u, 0x5342), 0x64806480u), d, h[1], l[1]);
      split_pair(f16x2_sub(__byte_perm(ub, 0x64646464u, 0x5140), 0x64806480u), d, h[2], l[2]);
      split_pair(f16x2_sub(__byte_perm(ub, 0x64646464u, 0x5342), 0x64806480u), d, h[3], l[3]);
    };
    uint32_t h[4], l[4];
    chunk(rr.q[0].x, rr.q[0].y, d0, h, l), sink.template put<0>(h, l);
    chunk(rr.q[0].z, rr.q[0].w, d0, h, l), sink.template put<1>(h, l);
    chunk(rr.q[1].x, rr.q[1].y, d0, h, l), sink.template put<2>(h, l);
    chunk(rr.q[1].z, rr.q[1].w, d0, h, l), sink.template put<3>(h, l);
    chunk(rr.q[2].x, rr.q[2].y, d1, h, l), sink.template put<4>(h, l);
    chunk(rr.q[2].z, rr.q[2].w, d1, h, l), sink.template put<5>(h, l);
    chunk(rr.q[3].x, rr.q[3].y, d1, h, l), sink.template put<6>(h, l);
    chunk(rr.q[3].z, rr.q[3].w, d1, h, l), sink.template put<7>(h, l);
  } else { // FC_Q4_0: nibbles p and p + 4 of a word are elements 2p and 2p + 1 (the 0x6400 / 0x5400 forms of dequant_q4_block)
    const RowRegs<FC_Q4_0>& rr = (const RowRegs<FC_Q4_0>&)r;
    const uint32_t d0 = scale_x2(rr.sc & 0xffffu, mul), d1 = scale_x2(rr.sc >> 16, mul);
    auto chunk = [&](uint32_t w, uint32_t d, uint32_t (&h)[4], uint32_t (&l)[4]) { // 8 nibbles
      const uint32_t w8 = w >> 8;
      split_pair(f16x2_sub((w & 0x000f000fu) | 0x64006400u, 0x64086408u), d, h[0], l[0]);  // 1024 + nib - 1032
      split_pair(f16x2_sub((w & 0x00f000f0u) | 0x54005400u, 0x54805480u), d, h[1], l[1]);  // 64 + nib - 72
      split_pair(f16x2_sub((w8 & 0x000f000fu) | 0x64006400u, 0x64086408u), d, h[2], l[2]);
      split_pair(f16x2_sub((w8 & 0x00f000f0u) | 0x54005400u, 0x54805480u), d, h[3], l[3]);
    };
    uint32_t h[4], l[4];
    chunk(rr.q[0].x, d0, h, l), sink.template put<0>(h, l);
    chunk(rr.q[0].y, d0, h, l), sink.template put<1>(h, l);
    chunk(rr.q[0].z, d0, h, l), sink.template put<2>(h, l);
    chunk(rr.q[0].w, d0, h, l), sink.template put<3>(h, l);
    chunk(rr.q[1].x, d1, h, l), sink.template put<4>(h, l);
    chunk(rr.q[1].y, d1, h, l), sink.template put<5>(h, l);
    chunk(rr.q[1].z, d1, h, l), sink.template put<6>(h, l);
    chunk(rr.q[1].w, d1, h, l), sink.template put<7>(h, l);
  }
}

struct TxArgs {
  uint32_t m = 0, n = 0, k = 0; // rows of x (<= 64), weight rows, width
  uint32_t mp = 64;             // rows of the xh and of the xl box: 16, 32 or 64 >= m (the MMAs' N is twice that)
  float* y = nullptr;           // [m][n]
  const float* bias = nullptr;  // [n]
  const float* resid = nullptr; // [m][n]; may alias y
  int act = ACT_NONE;
  int* err_flag = nullptr;
};

template <int KIND>
__global__ void __launch_bounds__(TX_THREADS, 1)
    qgemm_tx_kernel(const __grid_constant__ CUtensorMap tmap_xh, const __grid_constant__ CUtensorMap tmap_xl,
                    const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_sc, const TxArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u; // (the 128B swizzle is a function of the address)
  uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
  uint64_t* x_full = reinterpret_cast<uint64_t*>(smem + TX_X_STAGES * TX_STAGE_BYTES);
  uint64_t* x_empty = x_full + TX_X_STAGES;
  uint64_t* w_full = x_empty + TX_X_STAGES;
  uint64_t* acc_full = w_full + TX_W_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_word = tmem_slot + 1;
  float* unscale = reinterpret_cast<float*>(smem + TX_X_STAGES * TX_STAGE_BYTES + 512); // [4 chunks in flight][128 rows]: 2^-shift

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t k_iters = a.k / TC_BK;
  const uint32_t total_tiles = (a.n + TC_BN - 1) / TC_BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TX_X_STAGES; s++) {
      tc::mbar_init(&x_full[s], 1);
      tc::mbar_init(&x_empty[s], 1);
    }
    for (int t = 0; t < TX_W_STAGES; t++) {
      tc::mbar_init(&w_full[t], 4);
    }
    for (int b = 0; b < 2; b++) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 8);
    }
    *abort_word = 0;
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmap_xh);
    tc::prefetch_tmap(&tmap_xl);
    tc::prefetch_tmap(&tmap_q);
    tc::prefetch_tmap(&tmap_sc);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
    if (warp == 0) {
      // ---- TMA: per K step the x slices (the same for every tile: L2 after the first), the tile's packed weights
      // and the eight scales per row of the 256-k chunk the step lies in ----
      constexpr uint32_t STEP_BYTES = KIND == FC_Q8_0 ? 64 : 32;
      if (lane == 0) {
        uint32_t it = 0;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x) {
          for (uint32_t kk = 0; kk < k_iters; kk++, it++) {
            const uint32_t s = it % TX_X_STAGES, ph = (it / TX_X_STAGES) & 1;
            if (!wait_suspended(&x_empty[s], ph ^ 1, abort_word)) {
              atomicExch(a.err_flag, ERR_WAIT_EMPTY);
              break;
            }
            uint8_t* st = smem + s * TX_STAGE_BYTES;
            tc::mbar_arrive_expect_tx(&x_full[s], 2 * a.mp * 128 + TC_BN * STEP_BYTES + TC_BN * 16);
            tc::tma_load_2d(st, &tmap_xh, &x_full[s], (int32_t)(kk * TC_BK), 0);
            tc::tma_load_2d(st + a.mp * 128, &tmap_xl, &x_full[s], (int32_t)(kk * TC_BK), 0); // (a multiple of 1024: swizzle atoms stay whole)
            tc::tma_load_2d(st + TX_Q_OFF, &tmap_q, &x_full[s], (int32_t)(kk * STEP_BYTES), (int32_t)(tile * TC_BN));
            tc::tma_load_2d(st + TX_SC_OFF, &tmap_sc, &x_full[s], (int32_t)((kk / TX_CHUNK) * 16), (int32_t)(tile * TC_BN));
          }
        }
      }
    } else if (warp == 1) {
      // ---- MMA issuer: one elected thread runs the whole loop. What bounds this kernel is the chain of dependent
      // latencies in this loop (a satisfied mbarrier wait answers in about 200 cycles, a commit issues in about 80),
      // so it is kept to one wait and one commit per K step: w_full[t] implies the step's TMA bytes (the producers
      // waited for them), and one commit on x_empty[s] hands back the x stage and the weight stage together. ----
      if (tc::elect_one()) {
        const uint32_t idesc = a.mp == 64 ? tc::idesc_f16_f32(128, 128) : a.mp == 32 ? tc::idesc_f16_f32(128, 64) : tc::idesc_f16_f32(128, 32);
        constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29); // stride 1024 B, version 1, 128B swizzle
        uint32_t it = 0, ccnt = 0; // K steps and chunks issued so far
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
          for (uint32_t kc = 0; kc < k_iters && ok; kc += TX_CHUNK, ccnt++) {
            const uint32_t buf = ccnt & 1, aph = (ccnt >> 1) & 1;
            if (!wait_suspended(&acc_empty[buf], aph ^ 1, abort_word)) { // the epilogue has taken this buffer's last chunk
              atomicExch(a.err_flag, ERR_WAIT_ACC);
              ok = false;
              break;
            }
            tc::tc_fence_after();
            const uint32_t d1 = tmem_base + buf * TX_ACC_COLS;
            for (uint32_t kk = kc; kk < kc + TX_CHUNK; kk++, it++) {
              const uint32_t s = it % TX_X_STAGES, t = it % TX_W_STAGES;
              if (!wait_or_abort(&w_full[t], (it / TX_W_STAGES) & 1, abort_word)) {
                atomicExch(a.err_flag, ERR_WAIT_FULL);
                ok = false;
                break;
              }
              tc::tc_fence_after();
              const uint64_t dx = ((uint64_t)desc_hi << 32) | ((base + s * TX_STAGE_BYTES) >> 4);
              const uint32_t wh = tmem_base + TX_W_COL0 + t * TX_W_COLS, wl = wh + TX_W_COLS / 2;
              // eight MMAs of one shape into one accumulator (alternating shapes, or accumulators whose columns
              // overlap, run no faster)
#pragma unroll
              for (uint32_t ks = 0; ks < TC_BK / 16; ks++)
                tc::mma_f16_ts(d1, wh + ks * 8, dx + 2 * ks, idesc, (kk != kc || ks != 0) ? 1u : 0u); // wh . [xh | xl]; a chunk starts from zero
#pragma unroll
              for (uint32_t ks = 0; ks < TC_BK / 16; ks++) tc::mma_f16_ts(d1, wl + ks * 8, dx + 2 * ks, idesc, 1u); // + wl . [xh | xl]
              tc::mma_commit(&x_empty[s]);
            }
            if (ok) tc::mma_commit(&acc_full[buf]);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp < 4 + 4 * TX_PSETS) {
    // ---- weight producers (they and the epilogue warps keep the registers the CTA was launched with: about 100) ----
    const uint32_t pset = (uint32_t)(warp - 4) >> 2;
    const uint32_t quad = (uint32_t)warp & 3u;
    const uint32_t r = (quad << 5) + lane; // row of the tile = tensor-memory lane
    const uint32_t chunks = k_iters / TX_CHUNK;
    // where this thread's row lies in a stage's packed tile: 16-byte piece c of row r sits at piece c ^ (r / 2 % 4)
    // under the 64-byte swizzle (Q8_0 rows of 64 bytes), c ^ (r / 4 % 2) under the 32-byte one (Q4_0 rows of 32):
    // eight neighbouring rows read eight different bank groups
    constexpr uint32_t STEP_BYTES = KIND == FC_Q8_0 ? 64 : 32;
    const uint32_t sw = KIND == FC_Q8_0 ? ((r >> 1) & 3u) : ((r >> 2) & 1u);
    uint32_t tcnt = 0;
    float mul = 1.0f;
    for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x, tcnt++) {
      const uint32_t it0 = tcnt * k_iters;
      for (uint32_t kk = pset; kk < k_iters && !*abort_word; kk += TX_PSETS) {
        const uint32_t it = it0 + kk, t = it % TX_W_STAGES, s = it % TX_X_STAGES;
        if (!wait_suspended(&x_full[s], (it / TX_X_STAGES) & 1, abort_word)) {
          atomicExch(a.err_flag, ERR_WAIT_FULL);
          break;
        }
        const uint8_t* st = smem + s * TX_STAGE_BYTES;
        RowRegs<KIND> cur;
#pragma unroll
        for (uint32_t c = 0; c < STEP_BYTES / 16; c++)
          cur.q[c] = *reinterpret_cast<const uint4*>(st + TX_Q_OFF + r * STEP_BYTES + ((c ^ sw) << 4));
        const uint4 sc8 = *reinterpret_cast<const uint4*>(st + TX_SC_OFF + r * 16); // the chunk's eight scales
        const uint32_t scw[4] = {sc8.x, sc8.y, sc8.z, sc8.w};
        cur.sc = (kk & 2u) ? (pset ? sc8.w : sc8.z) : (pset ? sc8.y : sc8.x); // this step's two: word kk % 4
        static_assert(TX_CHUNK == 4 && TX_PSETS == 2, "the scale word select assumes steps pset, pset + 2 of a chunk of four");
        const bool opens = (kk % TX_CHUNK) == pset; // this set's first step of a chunk
        int shift = 0;
        if (opens) { // the power of two that brings the largest of the eight to [2^7, 2^8)
          float dmax = 0.0f;
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&scw[j]));
            dmax = fmaxf(dmax, fmaxf(fabsf(f.x), fabsf(f.y)));
          }
          if (dmax > 0.0f && dmax < INFINITY) shift = 7 - ((int)((__float_as_uint(dmax) >> 23) & 0xffu) - 127);
          mul = __uint_as_float((uint32_t)(127 + shift) << 23);
        }
        // the weight stage was last read by the MMAs of step it - 4, whose commit went to that step's x_empty
        if (it >= TX_W_STAGES &&
            !wait_suspended(&x_empty[(it - TX_W_STAGES) % TX_X_STAGES], ((it - TX_W_STAGES) / TX_X_STAGES) & 1, abort_word)) {
          atomicExch(a.err_flag, ERR_WAIT_EMPTY);
          break;
        }
        tc::tc_fence_after();
        if (opens && pset == 0) // (the slot's last reader, four chunks back, released its accumulator long before this stage emptied)
          unscale[((tcnt * chunks + kk / TX_CHUNK) & 3) * TC_BN + r] = __uint_as_float((uint32_t)(127 - shift) << 23);
        DualTmemSink sink;
        sink.taddr_hi = tmem_base + ((quad * 32u) << 16) + TX_W_COL0 + t * TX_W_COLS;
        sink.taddr_lo = sink.taddr_hi + TX_W_COLS / 2;
        emit_row_hilo<KIND>(cur, mul, sink);
        tc::tmem_st_wait();
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&w_full[t]);
      }
    }
  } else {
    // ---- epilogue: thread = output column n, 32 rows of x per warp ----
    const uint32_t e = warp - (4 + 4 * TX_PSETS), jhalf = e >> 2, quad = (uint32_t)warp & 3u;
    uint32_t tcnt = 0, ccnt = 0;
    bool ok = true;
    for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abort_word && ok; tile += gridDim.x, tcnt++) {
      const uint32_t n = tile * TC_BN + quad * 32 + lane;
      const bool n_ok = n < a.n;
      const float bias = (a.bias && n_ok) ? a.bias[n] : 0.0f;
      float acc[32];
#pragma unroll
      for (int j = 0; j < 32; j++) acc[j] = 0.0f;
      for (uint32_t kc = 0; kc < k_iters; kc += TX_CHUNK, ccnt++) {
        const uint32_t buf = ccnt & 1, aph = (ccnt >> 1) & 1;
        ok = wait_suspended(&acc_full[buf], aph, abort_word);
        if (!ok) atomicExch(a.err_flag, ERR_WAIT_ACC);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc::tc_fence_after();
        const float us = unscale[(ccnt & 3) * TC_BN + quad * 32 + lane]; // the chunk's power of two, divided out here
        // columns [0, mp) hold the products with xh, [mp, 2 mp) those with xl; this warp's rows of x are
        // [32 jhalf, 32 jhalf + 32) as far as they lie below mp
        const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + buf * TX_ACC_COLS + jhalf * 32;
#pragma unroll
        for (int c = 0; c < 2; c++) { // 16 rows of x at a time: two 16-column loads
          if (jhalf * 32 + c * 16 < a.mp) {
            uint32_t hh[16], sm[16];
            tc::tmem_ld_32x16(taddr + c * 16, hh);          // (wh + wl) . xh
            tc::tmem_ld_32x16(taddr + a.mp + c * 16, sm);   // (wh + wl) . xl
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; j++)
              acc[c * 16 + j] = fmaf(__uint_as_float(sm[j]) + __uint_as_float(hh[j]), us, acc[c * 16 + j]);
          }
        }
        // the chunk is in registers: the buffer may be refilled
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
      }
      if (!ok) break;
#pragma unroll
      for (int j = 0; j < 32; j++) {
        const uint32_t row = jhalf * 32 + j;
        float v = acc[j] + bias;
        if (a.act == ACT_GELU) v = gelu_f(v);
        if (n_ok && row < a.m) {
          const size_t at = (size_t)row * a.n + n;
          if (a.resid) v = a.resid[at] + v;
          a.y[at] = v;
        }
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
