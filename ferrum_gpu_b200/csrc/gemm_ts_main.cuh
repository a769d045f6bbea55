// The second kernel body of gemm_tc.cu (included there, inside its anonymous namespace): the product with the
// WEIGHT rows on the tensor-memory lanes.
//
//   D[n, x] = W[n, :] . X[x, :]      128 weight rows (lanes) x 192 activation rows (columns) per tile
//
// The dequantised weight slice never touches shared memory: a producer thread owns one weight row = one
// tensor-memory lane, turns the row's packed blocks of a 64-k slice into 32 columns of f16 pairs and writes them
// with tcgen05.st; the MMA takes them from there as its A operand (tcgen05.mma with A in tensor memory) and only
// the activation slice (192 rows x 128 bytes, one TMA box) is read from shared memory. Per MMA of 128 x 192 x 16
// that is 6 KB of shared-memory operand reads in 96 cycles, against 16 KB in 128 cycles when both operands of two
// 128 x 128 MMAs come from shared memory - the shared-memory pipe, which the TMA writes and the operand reads
// share, was what held that form at 0.6 of the tensor peak.
//
// The accumulator is the transposed output tile: a thread of the epilogue holds one output COLUMN n for 32
// consecutive output rows. A warp's 32 lanes are 32 consecutive columns, so every global access of the warp is
// one row's 128 contiguous bytes without a pass through shared memory; a per-column bias is one register; the
// gate / up pairs of SwiGLU sit on neighbouring lanes (weight rows 2i and 2i + 1) and meet by one shuffle.
//
// Tensor memory (512 columns): two accumulator buffers of 192 columns, four weight stages of 32 columns.
//
//   warp 0        TMA producer: one activation box per K step into a 6-deep ring
//   warp 1        tensor-memory owner and MMA issuer: 4 MMAs (K = 16) per K step
//   warps 4-15    weight producers in three sets of four warps (warp w owns lanes 32 (w % 4) ..); set p takes the
//                 K steps it with it % 3 == p. A producer's step is a chain of latencies (unpack, tcgen05.st and
//                 its wait, fence, arrive) of 1200-1800 cycles measured, against 400-500 for the MMAs of a step
//   warps 16-23   epilogue: warp w reads lane quadrant w % 4, columns [96 (w - 16) / 4, + 96)
//
// Barriers: x_full / x_empty (TMA bytes / MMA commit) for the activation ring, w_full / w_empty (4 producer-warp
// arrivals / MMA commit) for the weight stages, acc_full / acc_empty for the accumulator buffers. Every wait is
// bounded and polls the CTA-wide abort word.

template <int KIND, int EPI>
__global__ void __launch_bounds__(TS_THREADS, 1)
    qgemm_ts_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_o, const QMat w,
                    const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u; // (the 128B swizzle is a function of the address)
  uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
  uint64_t* x_full = reinterpret_cast<uint64_t*>(smem + X_STAGES * X_BYTES);
  uint64_t* x_empty = x_full + X_STAGES;
  uint64_t* w_full = x_empty + X_STAGES;
  uint64_t* w_empty = w_full + W_STAGES;
  uint64_t* acc_full = w_empty + W_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t k_iters = a.k / TC_BK;
  const uint32_t tiles_n = (a.n + TC_BN - 1) / TC_BN, tiles_x = (a.m + TS_BX - 1) / TS_BX;
  const uint32_t total_tiles = tiles_n * tiles_x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < X_STAGES; s++) {
      tc::mbar_init(&x_full[s], 1);
      tc::mbar_init(&x_empty[s], 1);
    }
    for (int t = 0; t < W_STAGES; t++) {
      tc::mbar_init(&w_full[t], 4);
      tc::mbar_init(&w_empty[t], 1);
    }
    for (int b = 0; b < 2; b++) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 8);
    }
    *abort_word = 0;
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmap_x);
    if (a.out_tma) tc::prefetch_tmap(&tmap_o);
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
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_CTRL));
    if (warp == 0) {
      // ---- TMA producer ----
      if (lane == 0) {
        uint32_t it = 0;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x) {
          const uint32_t x0 = (tile / tiles_n) * TS_BX;
          for (uint32_t kk = 0; kk < k_iters; kk++, it++) {
            const uint32_t s = it % X_STAGES, ph = (it / X_STAGES) & 1;
            if (!wait_or_abort(&x_empty[s], ph ^ 1, abort_word)) {
              atomicExch(a.err_flag, ERR_WAIT_EMPTY);
              break;
            }
            tc::mbar_arrive_expect_tx(&x_full[s], X_BYTES);
            tc::tma_load_2d(smem + s * X_BYTES, &tmap_x, &x_full[s], (int32_t)(kk * TC_BK), (int32_t)x0);
          }
        }
      }
    } else if (warp == 1) {
      // ---- MMA issuer: the whole warp waits (addresses stay warp-uniform), one elected lane issues ----
      const bool leader = tc::elect_one();
      constexpr uint32_t idesc = tc::idesc_f16_f32(128, TS_BX);
      constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29); // stride 1024 B, version 1, 128B swizzle
      uint32_t it = 0, tcnt = 0;
      bool ok = true;
      for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abort_word && ok; tile += gridDim.x, tcnt++) {
        const uint32_t buf = tcnt & 1, aph = (tcnt >> 1) & 1;
        if (!wait_or_abort(&acc_empty[buf], aph ^ 1, abort_word)) { // the epilogue has drained this buffer
          atomicExch(a.err_flag, ERR_WAIT_ACC);
          ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc::tc_fence_after();
        const uint32_t d = tmem_base + buf * TS_BX;
        for (uint32_t kk = 0; kk < k_iters; kk++, it++) {
          const uint32_t s = it % X_STAGES, t = it % W_STAGES;
          if (!wait_or_abort(&x_full[s], (it / X_STAGES) & 1, abort_word) ||
              !wait_or_abort(&w_full[t], (it / W_STAGES) & 1, abort_word)) {
            atomicExch(a.err_flag, ERR_WAIT_FULL);
            ok = false;
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc::tc_fence_after();
          const uint64_t dx = ((uint64_t)desc_hi << 32) | ((base + s * X_BYTES) >> 4);
          const uint32_t wa = tmem_base + W_COL0 + t * W_COLS;
          if (leader) {
#pragma unroll
            for (uint32_t ks = 0; ks < TC_BK / 16; ks++) // 16 k: 8 columns of the weight stage, 32 bytes of the swizzled row
              tc::mma_f16_ts(d, wa + ks * 8, dx + 2 * ks, idesc, (kk | ks) != 0 ? 1u : 0u);
            tc::mma_commit(&x_empty[s]);
            tc::mma_commit(&w_empty[t]);
          }
          __syncwarp();
        }
        if (!ok) break;
        if (leader) tc::mma_commit(&acc_full[buf]);
        __syncwarp();
      }
    }
  } else if (warp < 4 + 4 * PSETS) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TS_REGS_PROD));
    // ---- weight producers ----
    const uint32_t pset = (uint32_t)(warp - 4) >> 2;       // takes the K steps it with it % PSETS == pset
    const uint32_t quad = (uint32_t)warp & 3u;
    const uint32_t r = (quad << 5) + lane;                 // row of the 128-row weight slice = tensor-memory lane
    uint32_t tile = blockIdx.x, kk = 0, it = 0;
    auto step = [&](uint32_t& t_, uint32_t& k_) {
      if (++k_ == k_iters) {
        k_ = 0;
        t_ += gridDim.x;
      }
    };
    auto hop = [&](uint32_t& t_, uint32_t& k_) { // to the set's next step
#pragma unroll
      for (int i = 0; i < PSETS; i++) step(t_, k_);
    };
    for (uint32_t i = 0; i < pset; i++) step(tile, kk);
    it = pset;
    // The packed blocks are fetched several K steps before they are needed: the loads are 32-byte pieces of 128
    // different rows, served by L2 at several hundred cycles under load, and a producer that waits for them
    // stalls the tensor pipe. (Formats with large rows keep one step's distance: registers.)
    constexpr bool DEEP = sizeof(RowRegs<KIND>) <= 48;
    auto fetch = [&](RowRegs<KIND>& dst, uint32_t t_, uint32_t k_) {
      if (t_ < total_tiles) {
        const uint32_t row = (t_ % tiles_n) * TC_BN + r;
        load_row<KIND>(dst, w, row < w.n ? row : 0, k_, row < w.n);
      }
    };
    RowRegs<KIND> cur, nxt, far;
    uint32_t t1 = tile, k1 = kk; // the set's next step
    hop(t1, k1);
    uint32_t t2 = t1, k2 = k1;   // and the one after
    hop(t2, k2);
    fetch(cur, tile, kk);
    fetch(nxt, t1, k1);
    while (tile < total_tiles && !*abort_word) {
      const uint32_t t = it % W_STAGES, ph = (it / W_STAGES) & 1;
      if (DEEP) fetch(far, t2, k2);
      if (!wait_suspended(&w_empty[t], ph ^ 1, abort_word)) { // (suspended tries: twelve spinning warps cost the others issue slots)
        atomicExch(a.err_flag, ERR_WAIT_EMPTY);
        break;
      }
      tc::tc_fence_after(); // (the MMAs that read this stage are complete: seen through the barrier)
      TmemSink sink;
      sink.taddr = tmem_base + ((quad * 32u) << 16) + W_COL0 + t * W_COLS;
      emit_row<KIND>(cur, sink);
      tc::tmem_st_wait();
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&w_full[t]);
      cur = nxt;
      tile = t1, kk = k1;
      t1 = t2, k1 = k2;
      hop(t2, k2);
      it += PSETS;
      if (DEEP)
        nxt = far;
      else
        fetch(nxt, t1, k1);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TS_REGS_EPI));
    // ---- epilogue ----
    const uint32_t e = warp - (4 + 4 * PSETS), colhalf = e >> 2, quad = (uint32_t)warp & 3u;
    const bool odd = lane & 1;
    // Results leave through shared memory and TMA when the output can be a TMA tensor: the warp writes a chunk of
    // 32 rows x 32 columns as the row-major tile it is (lane = column: conflict-free), and one bulk tensor store -
    // for the residual stream a bulk tensor REDUCE (add), so the stream is never loaded - carries it out, clipped
    // at the matrix edges by the tensor map. Two staging tiles per warp: a tile is reused once the copy that read
    // it two chunks ago has finished reading.
    uint8_t* stage = smem + STG_OFF + e * (2 * STG_TILE);
    uint32_t sbuf = 0;
    uint32_t tcnt = 0;
    for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x, tcnt++) {
      const uint32_t buf = tcnt & 1, aph = (tcnt >> 1) & 1;
      const uint32_t n = (tile % tiles_n) * TC_BN + quad * 32 + lane; // this thread's output column
      const uint32_t x_first = (tile / tiles_n) * TS_BX + colhalf * (TS_BX / 2);
      const bool n_ok = n < a.n;
      const float bias = (a.bias && n_ok) ? a.bias[n] : 0.0f;
      const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + buf * TS_BX + colhalf * (TS_BX / 2);
      // The residual stream comes from DRAM. The lines this warp will add to in the CTA's NEXT tile are requested
      // into L2 now, a whole main loop ahead (a warp's 32 columns are one 128-byte line per row: three rows per
      // lane); this tile's values are then read 32 rows ahead of their use.
      float res[EPI == EPI_RESID ? 32 : 1];
      auto load_resid = [&](uint32_t x0) {
#pragma unroll
        for (int j = 0; j < 32; j++) res[j] = (n_ok && x0 + j < a.m) ? a.out_f32[(size_t)(x0 + j) * a.ldo + n] : 0.0f;
      };
      if (EPI == EPI_RESID && !a.out_tma) {
        const uint32_t nt = tile + gridDim.x;
        if (nt < total_tiles) {
          const uint32_t pn = (nt % tiles_n) * TC_BN + quad * 32, px = (nt / tiles_n) * TS_BX + colhalf * (TS_BX / 2);
#pragma unroll
          for (int i = 0; i < (int)(TS_BX / 64); i++) {
            const uint32_t row = px + i * 32 + lane;
            if (pn < a.n && row < a.m) asm volatile("prefetch.global.L2 [%0];" ::"l"(a.out_f32 + (size_t)row * a.ldo + pn));
          }
        }
        load_resid(x_first);
      }
      bool ok = wait_suspended(&acc_full[buf], aph, abort_word); // (the one long wait that is not on the tensor pipe's path)
      if (!ok) atomicExch(a.err_flag, ERR_WAIT_ACC);
      if (!__all_sync(0xffffffffu, ok)) break; // (the lanes leave together: the shuffles below take the whole warp)
      tc::tc_fence_after();
#pragma unroll 1
      for (uint32_t c = 0; c < TS_BX / 64; c++) {
        const uint32_t x0 = x_first + c * 32;
        uint32_t acc[32];
        tc::tmem_ld_32x32(taddr + c * 32, acc);
        tc::tmem_ld_wait();
        if (a.out_tma) {
          uint8_t* st = stage + sbuf * STG_TILE;
          sbuf ^= 1;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          if (EPI == EPI_F32 || EPI == EPI_RESID) {
            float* t = reinterpret_cast<float*>(st) + lane;
#pragma unroll
            for (int j = 0; j < 32; j++) t[j * 32] = __uint_as_float(acc[j]) + bias;
          } else if (EPI == EPI_F16) {
            __half* t = reinterpret_cast<__half*>(st) + lane;
#pragma unroll
            for (int j = 0; j < 32; j++) {
              float v = __uint_as_float(acc[j]) + bias;
              if (a.act == ACT_GELU) v = gelu_f(v);
              t[j * 32] = __ushort_as_half((unsigned short)(pack_f16(v, 0.0f) & 0xffffu));
            }
          } else { // SwiGLU: weight rows 2i / 2i + 1 are gate i / up i; the even lane finishes row j, the odd lane row j + 1
            __half* t = reinterpret_cast<__half*>(st) + (odd ? 16 : 0) + (lane >> 1);
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float got = __shfl_xor_sync(0xffffffffu, __uint_as_float(odd ? acc[j] : acc[j + 1]), 1);
              const float gv = odd ? got : __uint_as_float(acc[j]), uv = odd ? __uint_as_float(acc[j + 1]) : got;
              const float v = __fdividef(gv, 1.0f + ex2f_approx(gv * -1.4426950408889634f)) * uv;
              t[j * 16] = __ushort_as_half((unsigned short)(pack_f16(v, 0.0f) & 0xffffu));
            }
          }
          tc::fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int32_t col = (int32_t)((tile % tiles_n) * TC_BN + quad * 32) >> (EPI == EPI_SWIGLU ? 1 : 0);
            if (EPI == EPI_RESID)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&tmap_o),
                           "r"(tc::smem_u32(st)), "r"(col), "r"((int32_t)x0)
                           : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&tmap_o),
                           "r"(tc::smem_u32(st)), "r"(col), "r"((int32_t)x0)
                           : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        } else if (EPI == EPI_F32 || EPI == EPI_RESID) {
#pragma unroll
          for (int j = 0; j < 32; j++) {
            float v = __uint_as_float(acc[j]) + bias;
            if (EPI == EPI_RESID) v += res[j];
            if (n_ok && x0 + j < a.m) a.out_f32[(size_t)(x0 + j) * a.ldo + n] = v;
          }
          if (EPI == EPI_RESID && c + 1 < TS_BX / 64) load_resid(x0 + 32);
        } else if (EPI == EPI_F16) {
          // lanes 2i and 2i + 1 trade one of each pair of rows: the even lane stores row j of both columns, the
          // odd lane row j + 1 (n is a multiple of 8 on this path: a pair of columns is inside or outside together)
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float v0 = __uint_as_float(acc[j]) + bias, v1 = __uint_as_float(acc[j + 1]) + bias;
            if (a.act == ACT_GELU) v0 = gelu_f(v0), v1 = gelu_f(v1);
            const float got = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);
            const uint32_t pair = odd ? pack_f16(got, v1) : pack_f16(v0, got);
            const uint32_t row = x0 + j + (odd ? 1u : 0u);
            if (n_ok && row < a.m) *reinterpret_cast<uint32_t*>(a.out_f16 + (size_t)row * a.ldo + (n & ~1u)) = pair;
          }
        } else if (EPI == EPI_SWIGLU) {
          // weight rows 2i / 2i + 1 are gate i / up i: the even lane finishes row j, the odd lane row j + 1
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float got = __shfl_xor_sync(0xffffffffu, __uint_as_float(odd ? acc[j] : acc[j + 1]), 1);
            const float gv = odd ? got : __uint_as_float(acc[j]), uv = odd ? __uint_as_float(acc[j + 1]) : got;
            const float v = __fdividef(gv, 1.0f + ex2f_approx(gv * -1.4426950408889634f)) * uv;
            const uint32_t row = x0 + j + (odd ? 1u : 0u);
            if (n_ok && row < a.m) {
              const uint32_t h = pack_f16(v, 0.0f);
              a.out_f16[(size_t)row * a.ldo + (n >> 1)] = __ushort_as_half((unsigned short)(h & 0xffffu));
            }
          }
        }
      }
      // this warp's reads of the buffer are complete: hand it back to the MMA issuer
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); // the staged tiles are out before the CTA ends
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
