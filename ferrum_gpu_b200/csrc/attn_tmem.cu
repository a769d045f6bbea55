// Causal attention of the scoring path on the 5th-generation tensor cores: S = Q K^T and O = P V are
// tcgen05.mma instructions with their accumulators in tensor memory, Q / K / V tiles arrive by TMA
// straight from the packed [rows][q | k | v] fp16 buffer, and the softmax runs one query row per
// thread on tcgen05.ld'ed rows (no shuffles). Same contract as the mma.sync kernel in attn_tc.cu:
// replaces attn_gqa_scores.wgsl + attn_softmax.wgsl + attn_gqa_pv.wgsl
// (ferrum_wgpu/src/ops/llama.rs:L119-L146) without materialising the [t, t] probabilities.
//
// Persistent: one CTA per SM walks work items (sequence, head, block of 256 query rows), heaviest
// blocks first. An item's rows are two 128-row halves with their own accumulators, so the tensor pipe
// always has the other half's MMAs to run while one half's softmax warps are busy.
//
//   warp 0      TMA: the item's two Q halves, then its K and V tiles of 128 keys through a ring of KS
//               stages; runs ahead into the next item
//   warp 1      TMEM owner and MMA issuer (the warp walks the schedule, one elected lane issues), per
//               key tile j:  S0 = Q0 K_{j+1}^T | S1 = Q1 K_{j+1}^T  as soon as the scores of tile j are
//               in registers (they run under the softmax of tile j), then O0 += P0 V_j | O1 += P1 V_j
//   warps 4-7   softmax of half 0 (thread = query row): row max, p = 2^(s*c - m*c) as fp16 back into
//               tensor memory (the A operand of the P V product is read from there, so the
//               probabilities never touch shared memory), running sum,
//   warps 8-11  the same for half 1.   O accumulates in tensor memory over the key tiles; when a
//               row's maximum has moved by more than 2^8 the row's thread rescales its O row in
//               place (tcgen05.ld / st) once the previous P V has landed (pv_done).
//   setmaxnreg moves registers from warps 0-3 (56) to the softmax warps (224): a row's 128 scores
//   stay in registers from the maximum to the packed probabilities.
//
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,320) O1 [320,384) P0 [384,448) P1 [448,512)
// (P: two fp16 per 32-bit column).
// Barriers: q_full / q_empty[2] (TMA bytes / commit after the item's last S of the half),
// k_full / k_empty[KS], v_full / v_empty[KS] (TMA bytes / MMA commits), s_full[h] (commit after S_h),
// s_free[h] (4 softmax warps: the scores are in registers), p_full[h] (4 softmax warps: P_h written,
// O_h rescaled), pv_done[h] (commit after O_h += P_h V: P_h may be overwritten, O_h read or rescaled).
// Phases run on across items. Every wait is bounded and raises a CTA-wide abort word.
#include "gemm_tc.cuh"
#include "tc_ptx.cuh"

namespace {

constexpr int KS = 4;                 // K / V ring stages
constexpr int THREADS = 384;          // warps 0-3: TMA, MMA, two idle; warps 4-11 softmax (tcgen05.ld lane quarter = warp % 4)
constexpr uint32_t TILE_BYTES = 128 * 128; // 128 rows x 64 fp16
constexpr uint32_t OFF_Q = 0, OFF_K = 2 * TILE_BYTES, OFF_V = OFF_K + KS * TILE_BYTES;
constexpr uint32_t OFF_BAR = OFF_V + KS * TILE_BYTES;
constexpr uint32_t SMEM_BYTES = OFF_BAR + 512 + 1024; // + alignment slack
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_S = 0, COL_O = 256, COL_P = 384;
// setmaxnreg targets (4 control warps, 8 softmax warps). The pool is what the CTA was launched with
// (threads x registers per thread as compiled); an increase that does not fit waits forever, so the
// launch code checks the sum against the compiled register count first.
constexpr int REGS_CTRL = 56, REGS_SOFTMAX = 224;
constexpr int REGS_NEEDED = 32 * (4 * REGS_CTRL + 8 * REGS_SOFTMAX);
enum { ERR_ATTN_LOAD = 11, ERR_ATTN_MMA = 12, ERR_ATTN_SOFTMAX = 13 };

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_word) {
  for (uint32_t i = 0; i < tc::WAIT_LIMIT; i++) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_word) return false;
  }
  *abort_word = 1;
  return false;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// P V: A = P from tensor memory, B = V tile [keys][64] = N-major ("MN-major") operand, M 128 x N 64
__host__ __device__ constexpr uint32_t idesc_pv() { return tc::idesc_f16_f32(128, 64) | (1u << 16); }
// high word of a 128B-swizzle operand descriptor (stride 1024 B, version 1); the low word is address >> 4
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint64_t desc_at(uint32_t smem_addr) { return ((uint64_t)DESC_HI << 32) | (smem_addr >> 4); }

struct Item { // one (sequence, head, 256-row query block)
  uint32_t qb, h, seq, n0, n1, n_max;
};
__device__ __forceinline__ Item item_at(uint32_t w, uint32_t nqb, uint32_t heads, uint32_t n_seqs, uint32_t t) {
  Item it;
  const uint32_t per = heads * n_seqs;
  it.qb = nqb - 1 - w / per; // heaviest (latest) query blocks first
  const uint32_t hs = w % per;
  it.seq = hs / heads;
  it.h = hs % heads;
  // key tiles of each half: through its diagonal tile; half 1 is idle when it holds no row of the sequence
  it.n0 = 2 * it.qb + 1;
  it.n1 = (it.qb * 256 + 128 < t) ? 2 * it.qb + 2 : 0;
  it.n_max = it.n0 > it.n1 ? it.n0 : it.n1;
  return it;
}

__global__ void __launch_bounds__(THREADS, 1)
    attn_tmem_kernel(const __grid_constant__ CUtensorMap tmap, uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads,
                     __half* __restrict__ out, int* __restrict__ err_flag) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (tc::smem_u32(smem_raw) + 1023u) & ~1023u; // swizzle phase follows the absolute address
  uint8_t* smem = smem_raw + (base - tc::smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* q_full = bars;              // [2]  TMA bytes of a Q half
  uint64_t* q_empty = q_full + 2;       // [2]  commit after the item's last S of the half
  uint64_t* k_full = q_empty + 2;       // [KS]
  uint64_t* k_empty = k_full + KS;      // [KS]
  uint64_t* v_full = k_empty + KS;      // [KS]
  uint64_t* v_empty = v_full + KS;      // [KS]
  uint64_t* s_full = v_empty + KS;      // [2]  commit after S of the half
  uint64_t* s_free = s_full + 2;        // [2]  4 softmax warps: the scores are in registers
  uint64_t* p_full = s_free + 2;        // [2]  4 softmax warps: P written (and O rescaled)
  uint64_t* pv_done = p_full + 2;       // [2]  commit after O += P V of the half
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile uint32_t* abort_word = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t qd = heads * 64, kvd = kv_heads * 64, group = heads / kv_heads;
  const uint32_t nqb = (t + 255) / 256;
  const uint32_t n_items = nqb * heads * n_seqs;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; i++) {
      tc::mbar_init(&q_full[i], 1);
      tc::mbar_init(&q_empty[i], 1);
      tc::mbar_init(&s_full[i], 1);
      tc::mbar_init(&s_free[i], 4);
      tc::mbar_init(&p_full[i], 4);
      tc::mbar_init(&pv_done[i], 1);
    }
    for (int i = 0; i < KS; i++) {
      tc::mbar_init(&k_full[i], 1);
      tc::mbar_init(&k_empty[i], 1);
      tc::mbar_init(&v_full[i], 1);
      tc::mbar_init(&v_empty[i], 1);
    }
    *abort_word = (*err_flag != 0) ? 1u : 0u; // an earlier launch gave up: do not wait again
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmap);
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // 12 warps share the register file at 168 each; the softmax rows want their 128 scores in
  // registers, the copy and MMA warps need few: move the budget (56 + 2 x 224 <= 512 per lane slot)
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_CTRL));
    if (warp == 0) {
      // ---- TMA: runs ahead of the MMAs by the depth of the K / V ring, across work items ----
      if (lane == 0 && !*abort_word) {
        uint32_t g = 0;              // key tiles loaded so far (ring position)
        uint32_t qi[2] = {0, 0};     // Q halves loaded so far
        bool ok = true;
        for (uint32_t w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
          const Item it = item_at(w, nqb, heads, n_seqs, t);
          const uint32_t row_base = it.seq * t, q0 = it.qb * 256, kvh = it.h / group;
          for (uint32_t half = 0; half < 2; half++) {
            if (half == 1 && !it.n1) break;
            if (!wait_or_abort(&q_empty[half], (qi[half] & 1) ^ 1, abort_word)) { // the previous item's S reads are done
              ok = false;
              break;
            }
            qi[half]++;
            tc::mbar_arrive_expect_tx(&q_full[half], TILE_BYTES);
            tc::tma_load_2d(smem + OFF_Q + half * TILE_BYTES, &tmap, &q_full[half], (int32_t)(it.h * 64),
                            (int32_t)(row_base + q0 + half * 128));
          }
          for (uint32_t j = 0; j < it.n_max && ok; j++, g++) {
            const uint32_t s = g % KS, ph = (g / KS) & 1;
            if (!wait_or_abort(&k_empty[s], ph ^ 1, abort_word)) {
              ok = false;
              break;
            }
            tc::mbar_arrive_expect_tx(&k_full[s], TILE_BYTES);
            tc::tma_load_2d(smem + OFF_K + s * TILE_BYTES, &tmap, &k_full[s], (int32_t)(qd + kvh * 64),
                            (int32_t)(row_base + j * 128));
            if (!wait_or_abort(&v_empty[s], ph ^ 1, abort_word)) {
              ok = false;
              break;
            }
            tc::mbar_arrive_expect_tx(&v_full[s], TILE_BYTES);
            tc::tma_load_2d(smem + OFF_V + s * TILE_BYTES, &tmap, &v_full[s], (int32_t)(qd + kvd + kvh * 64),
                            (int32_t)(row_base + j * 128));
          }
        }
        if (!ok) atomicExch(err_flag, ERR_ATTN_LOAD);
      }
    } else if (warp == 1) {
      // ---- MMA issuer ----
      // The whole warp walks the schedule (addresses and descriptors stay warp-uniform); one elected
      // lane issues the MMAs and the commits.
      const bool leader = tc::elect_one();
      constexpr uint32_t idesc_s = tc::idesc_f16_f32(128, 128);
      constexpr uint32_t idesc_o = idesc_pv();
      bool ok = !*abort_word;
      auto wait = [&](uint64_t* bar, uint32_t parity) {
        if (ok && !wait_or_abort(bar, parity, abort_word)) {
          atomicExch(err_flag, ERR_ATTN_MMA);
          ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);
        tc::tc_fence_after();
        return ok;
      };
      auto commit = [&](uint64_t* bar) {
        if (leader) tc::mma_commit(bar);
        __syncwarp();
      };
      uint32_t cs[2] = {0, 0}; // S tiles issued per half since the kernel began (phase of s_full / s_free / p_full / pv_done)
      uint32_t cp[2] = {0, 0}; // P V products issued per half
      uint32_t ci[2] = {0, 0}; // items per half (phase of q_full)
      uint32_t g = 0;          // ring position of the item's key tile 0
      // S_half = Q_half K^T for the key tile in ring stage s; waits until the previous scores of the
      // half have been read into registers
      auto issue_s = [&](uint32_t half, uint32_t s) {
        if (!wait(&s_free[half], (cs[half] & 1) ^ 1)) return;
        cs[half]++;
        const uint64_t qa = desc_at(base + OFF_Q + half * TILE_BYTES), ka = desc_at(base + OFF_K + s * TILE_BYTES);
        if (leader) {
#pragma unroll
          for (uint32_t ks = 0; ks < 4; ks++) // 32 bytes = 16 fp16 along K inside the swizzled row
            tc::mma_f16(tmem_base + COL_S + half * 128, qa + ks * 2, ka + ks * 2, idesc_s, ks != 0 ? 1u : 0u);
          tc::mma_commit(&s_full[half]);
        }
        __syncwarp();
      };
      // O_half (+)= P_half V for the key tile in ring stage s, once the half's P is published
      auto issue_pv = [&](uint32_t half, uint32_t s, uint32_t first) {
        if (!wait(&p_full[half], cp[half] & 1)) return;
        cp[half]++;
        const uint64_t va = desc_at(base + OFF_V + s * TILE_BYTES);
        if (leader) {
#pragma unroll
          for (uint32_t ks = 0; ks < 8; ks++) // 16 keys: 8 columns of packed P, 16 rows (2048 bytes) of V
            tc::mma_f16_ts(tmem_base + COL_O + half * 64, tmem_base + COL_P + half * 64 + ks * 8, va + ks * 128, idesc_o,
                           (ks != 0 || !first) ? 1u : 0u);
          tc::mma_commit(&pv_done[half]);
        }
        __syncwarp();
      };
      for (uint32_t w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const Item it = item_at(w, nqb, heads, n_seqs, t);
        // the first scores of both halves
        if (!wait(&q_full[0], ci[0]++ & 1)) break;
        if (it.n1 && !wait(&q_full[1], ci[1]++ & 1)) break;
        if (!wait(&k_full[g % KS], (g / KS) & 1)) break;
        issue_s(0, g % KS);
        if (it.n0 == 1) commit(&q_empty[0]);
        if (it.n1) issue_s(1, g % KS);
        commit(&k_empty[g % KS]);
        // per key tile j: the scores of tile j + 1 as soon as tile j's are in registers (they run
        // under the softmax of tile j), then O += P_j V_j when P_j is published
        for (uint32_t j = 0; j < it.n_max && ok; j++) {
          const uint32_t gj = g + j, s = gj % KS, ph = (gj / KS) & 1;
          const uint32_t sn = (gj + 1) % KS, phn = ((gj + 1) / KS) & 1;
          const bool more0 = j + 1 < it.n0, more1 = j + 1 < it.n1;
          if (more0 || more1) {
            if (!wait(&k_full[sn], phn)) break;
            if (more0) {
              issue_s(0, sn);
              if (j + 2 == it.n0) commit(&q_empty[0]);
            }
            if (more1) {
              issue_s(1, sn);
              if (j + 2 == it.n1) commit(&q_empty[1]);
            }
            commit(&k_empty[sn]);
          }
          if (!wait(&v_full[s], ph)) break;
          if (j < it.n0) issue_pv(0, s, j == 0);
          if (j < it.n1) issue_pv(1, s, j == 0);
          commit(&v_empty[s]);
        }
        g += it.n_max;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    // ---- softmax, one query row per thread ----
    const uint32_t half = (warp - 4) >> 2, quad = warp & 3;
    const uint32_t r = quad * 32 + lane;             // row within the half = TMEM lane
    const uint32_t lane_base = tmem_base + ((quad * 32) << 16);
    const uint32_t s_addr = lane_base + COL_S + half * 128;
    const uint32_t o_addr = lane_base + COL_O + half * 64;
    const uint32_t p_addr = lane_base + COL_P + half * 64;
    const float sl2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
    uint32_t c = 0;                                  // key tiles of this half since the kernel began
    bool ok = !*abort_word;
    for (uint32_t w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
      const Item it = item_at(w, nqb, heads, n_seqs, t);
      const uint32_t n_tiles = half ? it.n1 : it.n0;
      const uint32_t diag = 2 * it.qb + half;        // the one key tile that needs the causal mask
      float m_run = -INFINITY, l_run = 0.0f;
      for (uint32_t j = 0; j < n_tiles && ok; j++, c++) {
        if (!wait_or_abort(&s_full[half], c & 1, abort_word)) {
          ok = false;
          break;
        }
        tc::tc_fence_after();
        uint32_t v[128]; // this row's 128 scores; the packed probabilities replace them in place
#pragma unroll
        for (int q = 0; q < 4; q++) tc::tmem_ld_32x32(s_addr + q * 32, v + 32 * q);
        tc::tmem_ld_wait();
        // the scores are in registers: the tensor pipe may overwrite them with the next tile's
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&s_free[half]);
        if (j == diag) {
#pragma unroll
          for (int i = 0; i < 128; i++)
            if ((uint32_t)i > r) v[i] = 0xff800000u; // -inf: keys after this row's position
        }
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
          mx[0] = fmaxf(mx[0], __uint_as_float(v[i]));
          mx[1] = fmaxf(mx[1], __uint_as_float(v[i + 1]));
          mx[2] = fmaxf(mx[2], __uint_as_float(v[i + 2]));
          mx[3] = fmaxf(mx[3], __uint_as_float(v[i + 3]));
        }
        // key 0 of tile 0 is visible to every row, so the running maximum is finite from tile 0 on
        const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])));
        // Lazy rescale: the reference point of the exponentials moves only when some row of the warp
        // gained more than 2^8 over it (always at tile 0); until then probabilities may exceed 1 by
        // that factor, which fp16 and the f32 sums hold without loss.
        const bool moved = (m_new - m_run) * sl2 > 8.0f;
        bool pv_seen = false; // whether the previous P V of this half is known to be complete
        if (__any_sync(0xffffffffu, moved)) {
          const float corr = ex2((m_run - m_new) * sl2);
          m_run = m_new;
          l_run *= corr;
          if (j > 0) {
            if (!wait_or_abort(&pv_done[half], (c & 1) ^ 1, abort_word)) { // O must be at rest
              ok = false;
              break;
            }
            tc::tc_fence_after();
            pv_seen = true;
            uint32_t ov[32];
#pragma unroll
            for (int q = 0; q < 2; q++) {
              tc::tmem_ld_32x32(o_addr + q * 32, ov);
              tc::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; i++) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * corr);
              tc::tmem_st_32x32(o_addr + q * 32, ov);
            }
          }
        }
        const float msc = m_run * sl2;
        float ls[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(v[i]), sl2, -msc));
          const float p1 = ex2(fmaf(__uint_as_float(v[i + 1]), sl2, -msc));
          ls[(i >> 1) & 3] += p0 + p1;
          v[i >> 1] = pack_f16(p0, p1);
        }
        l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        // the previous P V of this half still reads the P columns: it has had a whole softmax to finish
        if (!pv_seen && c > 0) {
          if (!wait_or_abort(&pv_done[half], (c & 1) ^ 1, abort_word)) {
            ok = false;
            break;
          }
          tc::tc_fence_after();
        }
        tc::tmem_st_32x32(p_addr, v);
        tc::tmem_st_32x32(p_addr + 32, v + 32);
        tc::tmem_st_wait();
        // O rescaled and P written: publish to the tensor pipe
        tc::tc_fence_before();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&p_full[half]);
      }
      if (ok && n_tiles) { // the item's last P V, then normalise and store this row
        if (!wait_or_abort(&pv_done[half], (c & 1) ^ 1, abort_word)) {
          ok = false;
          break;
        }
        tc::tc_fence_after();
        uint32_t ov[64];
        tc::tmem_ld_32x32(o_addr, ov);
        tc::tmem_ld_32x32(o_addr + 32, ov + 32);
        tc::tmem_ld_wait();
        const uint32_t qrow = it.qb * 256 + half * 128 + r;
        if (qrow < t) {
          const float inv = 1.0f / l_run;
          uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)it.seq * t + qrow) * qd + it.h * 64);
#pragma unroll
          for (int q = 0; q < 8; q++) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = __uint_as_float(ov[8 * q + i]) * inv;
            dst[q] = make_uint4(pack_f16(f[0], f[1]), pack_f16(f[2], f[3]), pack_f16(f[4], f[5]), pack_f16(f[6], f[7]));
          }
        }
      }
    }
    if (!ok) atomicExch(err_flag, ERR_ATTN_SOFTMAX);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

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

} // namespace

bool attn_tmem_supports(uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads, uint32_t hd) {
  return hd == 64 && kv_heads && heads % kv_heads == 0 && n_seqs <= 65535 && heads <= 65535 &&
         (uint64_t)n_seqs * t < 0x7fffff00ull;
}

int k_attn_causal_tmem(FcDevice* dev, const __half* qkv, uint32_t n_seqs, uint32_t t, uint32_t heads, uint32_t kv_heads,
                       uint32_t hd, __half* out) {
  if (!n_seqs || !t) return FC_OK;
  if (!attn_tmem_supports(n_seqs, t, heads, kv_heads, hd))
    return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensor-memory attention needs head_dim 64 and at most 65535 sequences");
  if ((reinterpret_cast<uintptr_t>(qkv) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return fc_fail(dev, FC_ERR_ARG, "attention buffers must be 16-byte aligned");
  EncodeTiledFn enc = encode_fn();
  if (!enc) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const uint64_t width = (uint64_t)(heads + 2 * kv_heads) * 64;
  CUtensorMap tmap;
  const cuuint64_t dims[2] = {width, (cuuint64_t)n_seqs * t};
  const cuuint64_t strides[1] = {width * 2};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void*)qkv, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fc_fail(dev, FC_ERR_DEVICE, "cuTensorMapEncodeTiled failed with %d", (int)cr);
  static OncePerDevice attr;
  if (attr.first(dev->ordinal)) {
    attr.again(dev->ordinal); // (until the checks below have passed)
    cudaFuncAttributes fa;
    FC_CUDA(dev, cudaFuncGetAttributes(&fa, attn_tmem_kernel));
    if (fa.numRegs * THREADS < REGS_NEEDED)
      return fc_fail(dev, FC_ERR_UNSUPPORTED, "the tensor-memory attention was compiled with %d registers per thread; its "
                     "register rebalancing needs %d", fa.numRegs, (REGS_NEEDED + THREADS - 1) / THREADS);
    FC_CUDA(dev, cudaFuncSetAttribute(attn_tmem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    attr.first(dev->ordinal);
  }
  // persistent: one CTA per SM walks the (query block, sequence, head) items, heaviest blocks first
  const uint64_t items = (uint64_t)((t + 255) / 256) * heads * n_seqs;
  if (items > 0x7fffffffull) return fc_fail(dev, FC_ERR_UNSUPPORTED, "too many attention work items for one launch");
  const uint32_t sms = (uint32_t)dev->prop.multiProcessorCount;
  dim3 grid((unsigned)(items < sms ? items : sms));
  FC_LAUNCH(dev, "attn_causal_tmem",
            attn_tmem_kernel<<<grid, THREADS, SMEM_BYTES, dev->stream>>>(tmap, n_seqs, t, heads, kv_heads, out, dev->d_flag));
  return FC_OK;
}
