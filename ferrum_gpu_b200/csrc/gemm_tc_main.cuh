// The kernel body of gemm_tc.cu (included there, inside its anonymous namespace).

template <int KIND, int EPI>
__global__ void __launch_bounds__(THREADS, 2)
    qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const QMat w, const TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B swizzle is a function of the absolute shared-memory address
  const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * TC_BN, m0 = blockIdx.y * TC_BM;
  const uint32_t k_iters = a.k / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      tc::mbar_init(&full[s], 1 + 4); // TMA thread (with its byte count) + one arrive per weight-producer warp
      tc::mbar_init(&empty[s], 1);    // the MMA thread's commit
    }
    tc::mbar_init(acc_full, 1);
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmap_a);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, TC_BN);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      for (uint32_t it = 0; it < k_iters; it++) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
        if (!tc::mbar_wait(&empty[s], ph ^ 1)) {
          atomicExch(a.err_flag, ERR_WAIT_EMPTY);
          break;
        }
        tc::mbar_arrive_expect_tx(&full[s], A_BYTES);
        tc::tma_load_2d(smem + s * STAGE_BYTES, &tmap_a, &full[s], (int32_t)(it * TC_BK), (int32_t)m0);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc = tc::idesc_bf16_f32(TC_BM, TC_BN);
      bool ok = true;
      for (uint32_t it = 0; it < k_iters && ok; it++) {
        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
        if (!tc::mbar_wait(&full[s], ph)) {
          atomicExch(a.err_flag, ERR_WAIT_FULL);
          ok = false;
          break;
        }
        tc::tc_fence_after();
        const uint32_t a_addr = base + s * STAGE_BYTES, b_addr = a_addr + A_BYTES;
#pragma unroll
        for (uint32_t ks = 0; ks < TC_BK / 16; ks++) {
          const uint64_t da = tc::smem_desc_sw128(a_addr + ks * 32);
          const uint64_t db = tc::smem_desc_sw128(b_addr + ks * 32);
          tc::mma_bf16(tmem_base, da, db, idesc, (it | ks) != 0 ? 1u : 0u);
        }
        tc::mma_commit(&empty[s]); // the slice can be refilled once these MMAs have read it
      }
      tc::mma_commit(acc_full);    // accumulator complete (or abandoned: the epilogue must not hang)
    }
  } else {
    // ---- weight producers, then epilogue ----
    const uint32_t r = threadIdx.x - 64;        // weight row of the tile owned by this thread
    const uint32_t row = n0 + r;
    const bool valid = row < w.n;
    const uint32_t sw = r & 7;
    RowRegs<KIND> cur, nxt;
    load_row<KIND>(cur, w, valid ? row : 0, 0, valid);
    bool ok = true;
    for (uint32_t it = 0; it < k_iters; it++) {
      const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
      if (it + 1 < k_iters) load_row<KIND>(nxt, w, valid ? row : 0, it + 1, valid);
      if (!tc::mbar_wait(&empty[s], ph ^ 1)) {
        atomicExch(a.err_flag, ERR_WAIT_EMPTY);
        ok = false;
        break;
      }
      store_row<KIND>(cur, base + s * STAGE_BYTES + A_BYTES + r * 128, sw);
      tc::fence_async_smem();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&full[s]);
      cur = nxt;
    }
    // epilogue: this warp may read TMEM lanes [32 * (warp % 4), +32)
    const uint32_t quad = warp & 3;
    const uint32_t out_row = m0 + quad * 32 + lane;
    if (ok && !tc::mbar_wait(acc_full, 0)) {
      atomicExch(a.err_flag, ERR_WAIT_ACC);
      ok = false;
    }
    tc::tc_fence_after();
    if (ok) {
      const uint32_t taddr = tmem_base + ((quad * 32) << 16);
      if (EPI == EPI_SWIGLU) {
        // columns [0, 64) of the tile are gate rows, [64, 128) the matching up rows
#pragma unroll 1
        for (uint32_t c = 0; c < 2; c++) {
          uint32_t g[32], u[32];
          tc::tmem_ld_32x32(taddr + c * 32, g);
          tc::tmem_ld_32x32(taddr + 64 + c * 32, u);
          tc::tmem_ld_wait();
          epilogue_swiglu(a, out_row, (n0 / 2) + c * 32, g, u);
        }
      } else if (EPI == EPI_LSE) {
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
          *reinterpret_cast<float4*>(a.partial + ((size_t)blockIdx.x * a.m + out_row) * 4) =
              make_float4(st.mx, st.se, st.tl, (float)st.first);
      } else {
#pragma unroll 1
        for (uint32_t c = 0; c < TC_BN / 32; c++) {
          uint32_t acc[32];
          tc::tmem_ld_32x32(taddr + c * 32, acc);
          tc::tmem_ld_wait();
          epilogue_chunk<EPI>(a, out_row, n0 + c * 32, acc);
        }
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, TC_BN);
  }
}
