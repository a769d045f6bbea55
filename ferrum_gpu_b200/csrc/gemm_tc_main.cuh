// The first kernel body of gemm_tc.cu (included there, inside its anonymous namespace): the product with the
// ACTIVATION rows on the tensor-memory lanes, kept for the vocabulary head's log-sum-exp epilogue, where a thread
// folds one row's logits (max, sum of exponentials, target logit, first argmax) in its registers.
//
// Persistent: one CTA per SM walks output tiles of 256 x 128 (two 128-row accumulators that share
// one dequantised weight slice, which halves the dequantisation work per MMA). Tensor memory holds
// two such tiles (4 x 128 columns), so the epilogue of tile i overlaps the main loop of tile i+1.
//
//   warp 0        TMA producer: A slice, 256 rows x 64 f16 = one 32 KB swizzled box per K step
//   warp 1        TMEM owner and MMA issuer: 2 accumulators x 4 MMAs (K = 16) per K step
//   warps 4-7     weight producers of the even K steps: one weight row per thread, packed blocks ->
//   warps 8-11    f16 swizzled slice in shared memory; the same for the odd K steps. A producer's step is a
//                 chain of latencies (wait for the stage, dequantise, proxy fence, arrive) longer than the MMAs
//                 of a step, so two sets leapfrog.
//   warps 12-19   epilogue: warp w reads TMEM lane quadrant w % 4 of accumulator (w - 12) / 4
//   (warps 2-3 idle: roles are aligned to groups of four warps so that setmaxnreg can move registers
//   from the copy / MMA / producer warps to the epilogue warps)
//
// Barriers: full[s] (TMA bytes + 4 producer-warp arrivals) / empty[s] (MMA commit) for the
// shared-memory ring; acc_full[b] (MMA commit) / acc_empty[b] (8 epilogue-warp arrivals) for the two
// accumulator buffers. Every wait is bounded; the first wait that gives up raises a CTA-wide abort
// word that every loop polls, so a protocol error ends the kernel within one bounded wait.

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word) {
  for (uint32_t i = 0; i < tc::WAIT_LIMIT; i++) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_word) return false;
  }
  *abort_word = 1;
  return false;
}

// Bounded wait with suspended tries of up to 20 us each (about 1.3 s in all); polls the CTA's abort word.
__device__ __forceinline__ bool wait_suspended(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word) {
  for (uint32_t i = 0; i < (1u << 16); i++) {
    if (tc::mbar_try_wait_for(bar, parity, 20000u)) return true;
    if (*abort_word) return false;
  }
  *abort_word = 1;
  return false;
}

template <int KIND, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
    qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const QMat w, const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B swizzle is a function of the absolute shared-memory address
  const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t k_iters = a.k / TC_BK;
  const uint32_t tiles_n = (a.n + TC_BN - 1) / TC_BN, tiles_m = (a.m + TC_BM - 1) / TC_BM;
  const uint32_t total_tiles = tiles_n * tiles_m;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      tc::mbar_init(&full[s], 1 + 4);
      tc::mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 8);
    }
    *abort_word = 0;
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmap_a);
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
        const uint32_t m0 = (tile / tiles_n) * TC_BM;
        for (uint32_t kk = 0; kk < k_iters; kk++, it++) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!wait_or_abort(&empty[s], ph ^ 1, abort_word)) {
            atomicExch(a.err_flag, ERR_WAIT_EMPTY);
            break;
          }
          tc::mbar_arrive_expect_tx(&full[s], A_BYTES);
          tc::tma_load_2d(smem + s * STAGE_BYTES, &tmap_a, &full[s], (int32_t)(kk * TC_BK), (int32_t)m0);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    // The whole warp walks the tiles and waits (addresses and descriptors stay warp-uniform, which
    // keeps the per-instruction issue cost low); one elected lane issues the MMAs and the commits.
    const bool leader = tc::elect_one();
    constexpr uint32_t idesc = tc::idesc_f16_f32(128, TC_BN);
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
      const uint32_t d0 = tmem_base + buf * (2 * TC_BN), d1 = d0 + TC_BN;
      for (uint32_t kk = 0; kk < k_iters; kk++, it++) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
        if (!wait_or_abort(&full[s], ph, abort_word)) {
          atomicExch(a.err_flag, ERR_WAIT_FULL);
          ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc::tc_fence_after();
        const uint32_t a_addr = base + s * STAGE_BYTES;
        const uint64_t da0 = ((uint64_t)desc_hi << 32) | (a_addr >> 4);
        const uint64_t da1 = ((uint64_t)desc_hi << 32) | ((a_addr + A_BYTES / 2) >> 4);
        const uint64_t db = ((uint64_t)desc_hi << 32) | ((a_addr + A_BYTES) >> 4);
        if (leader) {
#pragma unroll
          for (uint32_t ks = 0; ks < TC_BK / 16; ks++) { // 32 bytes = 16 f16 along K inside the swizzled row
            tc::mma_f16(d0, da0 + 2 * ks, db + 2 * ks, idesc, (kk | ks) != 0 ? 1u : 0u);
            tc::mma_f16(d1, da1 + 2 * ks, db + 2 * ks, idesc, (kk | ks) != 0 ? 1u : 0u);
          }
          tc::mma_commit(&empty[s]);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (leader) tc::mma_commit(&acc_full[buf]);
      __syncwarp();
    }
  }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_PROD));
    // ---- weight producers ----
    const uint32_t pset = (uint32_t)(warp - 4) >> 2;     // 0: even K steps, 1: odd K steps
    const uint32_t r = ((uint32_t)(warp & 3) << 5) + lane; // row of the 128-row weight slice
    const uint32_t sw = r & 7;
    // this set's position in the CTA's sequence of (tile, K step) pairs
    uint32_t tile = blockIdx.x, kk = 0, it = 0;
    auto step = [&](uint32_t& t_, uint32_t& k_) {
      if (++k_ == k_iters) {
        k_ = 0;
        t_ += gridDim.x;
      }
    };
    if (pset) {
      step(tile, kk);
      it = 1;
    }
    RowRegs<KIND> cur, nxt;
    if (tile < total_tiles) {
      const uint32_t row = (tile % tiles_n) * TC_BN + r;
      load_row<KIND>(cur, w, row < w.n ? row : 0, kk, row < w.n);
    }
    while (tile < total_tiles && !*abort_word) {
      const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
      // prefetch the packed blocks of this set's next K step (two steps on, possibly in a later tile)
      uint32_t ntile = tile, nkk = kk;
      step(ntile, nkk);
      step(ntile, nkk);
      if (ntile < total_tiles) {
        const uint32_t nrow = (ntile % tiles_n) * TC_BN + r;
        load_row<KIND>(nxt, w, nrow < w.n ? nrow : 0, nkk, nrow < w.n);
      }
      if (!wait_suspended(&empty[s], ph ^ 1, abort_word)) {
        atomicExch(a.err_flag, ERR_WAIT_EMPTY);
        break;
      }
      SmemSink sink{base + s * STAGE_BYTES + A_BYTES + r * 128, sw};
      emit_row<KIND>(cur, sink);
      tc::fence_async_smem();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&full[s]);
      cur = nxt;
      tile = ntile;
      kk = nkk;
      it += 2;
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_EPI));
    // ---- epilogue ----
    const uint32_t e = warp - 12, half = e >> 2, quad = warp & 3;
    uint32_t tcnt = 0;
    for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abort_word; tile += gridDim.x, tcnt++) {
      const uint32_t buf = tcnt & 1, aph = (tcnt >> 1) & 1;
      const uint32_t n0 = (tile % tiles_n) * TC_BN;
      const uint32_t out_row = (tile / tiles_n) * TC_BM + half * 128 + quad * 32 + lane;
      if (!wait_suspended(&acc_full[buf], aph, abort_word)) {
        atomicExch(a.err_flag, ERR_WAIT_ACC);
        break;
      }
      tc::tc_fence_after();
      const uint32_t taddr = tmem_base + ((quad * 32) << 16) + buf * (2 * TC_BN) + half * TC_BN;
      { // the head's online log-sum-exp: this thread folds its row's 128 logits of the tile in registers
        LseState st;
        const int target = out_row < a.m ? a.targets[out_row] : -1;
#pragma unroll 1
        for (uint32_t c = 0; c < TC_BN / 32; c++) {
          uint32_t acc[32];
          tc::tmem_ld_32x32(taddr + c * 32, acc);
          tc::tmem_ld_wait();
          epilogue_lse(a, st, n0 + c * 32, target, acc);
        }
        if (out_row < a.m)
          *reinterpret_cast<float4*>(a.partial + ((size_t)(tile % tiles_n) * a.m + out_row) * 4) =
              make_float4(st.mx, st.se, st.tl, (float)st.first);
      }
      // this warp's reads of the buffer are complete: hand it back to the MMA issuer
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
