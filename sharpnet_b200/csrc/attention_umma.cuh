// Scaled dot-product attention forward as ONE tcgen05 kernel (3xTF32):
//
//   weights = softmax(mask(scaling * Q K^T)),  y = weights V          per matrix of the batch
//
// for score rows that fit one tile: v_steps <= 128 and embedding_dim <= 128.  One persistent CTA per SM walks over
// work units (matrix b, block of 128 query rows).  Per unit:
//   phase 1   S [128 x TKN] = Q K^T: both operands stream through the shared-memory ring in 32-deep K blocks, the
//             split warps add their lo planes, the tensor core accumulates the three TF32 products in TMEM;
//   softmax   the four epilogue warps (one score row per lane) read S from TMEM, apply scaling, the causal overwrite
//             with -1e12 and the softmax, and write the probabilities back to TMEM as the A operand of the second
//             product -- raw over S (the tensor core truncates to TF32 itself) and lo = tf32(p - hi) beside it --
//             then store them to `weights` (the layer keeps them for its backward pass) while the tensor core works;
//   phase 2   O [128 x EN] = P V with P read from TMEM (A operand in tensor memory) and V streamed through the same
//             ring as an MN-major B tile with its lo plane; the epilogue warps store O as y.
// The ring runs on across units, so the loads (and the first product) of the next unit overlap the softmax, the
// second product and the stores of the current one.  No scores buffer and no second launch.
//
// Reference: ScaledDotProductAttentionLayer.ScaledDotProductAttentionForwardPropagation
// (Prod/Layers/ScaledDotProductAttentionLayer.cs:46-91).
#pragma once
#include "gemm_umma.cuh"

namespace snb {

template <int TKN_, int EN_>
struct AttnTile {
  static constexpr int TKN = TKN_;                       // score columns (v_steps padded): N of phase 1, K of phase 2
  static constexpr int EN = EN_;                         // embedding columns padded: K of phase 1, N of phase 2
  static constexpr int BK = 32;
  static constexpr int Q_BYTES = 128 * BK * 4;           // phase-1 A block
  static constexpr int K_BYTES = TKN * BK * 4;           // phase-1 B block
  static constexpr int RAW1 = Q_BYTES + K_BYTES;
  static constexpr int RAW2 = EN * BK * 4;               // phase-2 B block: 32 rows of V
  static constexpr int STAGE1 = 2 * RAW1, STAGE2 = 2 * RAW2;   // raw tiles + lo planes
  static constexpr int STAGE_BYTES = STAGE1 > STAGE2 ? STAGE1 : STAGE2;
  static constexpr int STAGES_RAW = (192 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;
  static constexpr int SMEM_BYTES = RING_BYTES + 4 * EPI_STAGE_BYTES + 1024;
  static constexpr int THREADS = 384;                    // 4 control warps, 4 epilogue warps, 4 split warps
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S = 0, COL_PLO = TKN, COL_O = 2 * TKN;   // TMEM columns
  static constexpr int REGS_CTRL = 72, REGS_SPLIT = 64, REGS_EPI = 232;
  static constexpr int REGS_LAUNCH = (65536 / THREADS) / 8 * 8;   // what the CTA is launched with, per thread
  static_assert(REGS_CTRL + REGS_SPLIT + REGS_EPI <= THREADS / 128 * REGS_LAUNCH, "register shares exceed the CTA's pool");
  static constexpr int MN_CHUNK_BYTES = BK * 128;
  static_assert(TKN == 32 || TKN == 64 || TKN == 128, "score tile 32, 64 or 128 wide");
  static_assert(EN == 32 || EN == 64 || EN == 128, "embedding tile 32, 64 or 128 wide");
  static_assert(STAGES >= 2, "need two stages");
  static_assert(2 * TKN + EN <= 512, "TMEM columns");
};

struct AttnParams {
  int batch, q_steps, v_steps, embedding_dim;
  int tiles_q;            // blocks of 128 query rows per matrix
  UmmaParams s;           // placement of `weights` [batch, q_steps, v_steps], scaling in alpha, causal, row_op
  UmmaParams o;           // placement of y [batch, q_steps, embedding_dim] (possibly mapped)
  int* error_word;
};

template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  constexpr int TKN = T::TKN, EN = T::EN, BK = T::BK, STAGES = T::STAGES;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[STAGES], split_bar[STAGES], empty_bar[STAGES];
  __shared__ uint64_t s_full_bar, p_ready_bar, o_full_bar, o_empty_bar;
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;
  __shared__ float row_xch[1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* ring = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&split_bar[s], 4);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&s_full_bar, 1);
    mbar_init(&p_ready_bar, 4);
    mbar_init(&o_full_bar, 1);
    mbar_init(&o_empty_bar, 4);
    abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_holder, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_holder;
  volatile int* abortp = &abort_flag;
  allow_dependent_launch();
  grid_dependency_wait();

  const int units = p.batch * p.tiles_q;
  const int kb1 = (p.embedding_dim + BK - 1) / BK;       // K blocks of phase 1
  const int kb2 = (p.v_steps + BK - 1) / BK;             // K blocks of phase 2

  if (warp < 4) {
    reg_dealloc<T::REGS_CTRL>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int b = u / p.tiles_q, m0 = (u - b * p.tiles_q) * 128;
        for (int kb = 0; kb < kb1 + kb2; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) { ok = false; break; }
          uint8_t* dst = ring + s * T::STAGE_BYTES;
          if (kb < kb1) {
            mbar_arrive_expect_tx(&full_bar[s], T::RAW1);
            tma_load_3d(dst, &tmQ, &full_bar[s], kb * BK, m0, b);
            tma_load_3d(dst + T::Q_BYTES, &tmK, &full_bar[s], kb * BK, 0, b);
          } else {
            mbar_arrive_expect_tx(&full_bar[s], T::RAW2);
#pragma unroll
            for (int j = 0; j < EN / 32; ++j)
              tma_load_3d(dst + j * T::MN_CHUNK_BYTES, &tmV, &full_bar[s], 32 * j, (kb - kb1) * BK, b);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      const uint32_t idesc1 = make_idesc_tf32(128, TKN, 0, 0);
      const uint32_t idesc2 = make_idesc_tf32(128, EN, 0, 1);
      int s = 0;
      uint32_t ph = 0, it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++it) {
        // phase 1: S = Q K^T.  S is free: the products of the previous unit that read P from these columns were
        // issued before, and the tensor core runs what one thread issues in order.
        for (int kb = 0; kb < kb1; ++kb) {
          if (!mbar_wait(&split_bar[s], ph, abortp)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_hi = smem_u32(ring + s * T::STAGE_BYTES), b_hi = a_hi + T::Q_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / kUmmaK; ++ks) {
            const uint64_t da_hi = make_smem_desc(a_hi + ks * 32, 16, 1024, 2);
            const uint64_t db_hi = make_smem_desc(b_hi + ks * 32, 16, 1024, 2);
            const uint64_t da_lo = make_smem_desc(a_hi + T::RAW1 + ks * 32, 16, 1024, 2);
            const uint64_t db_lo = make_smem_desc(b_hi + T::RAW1 + ks * 32, 16, 1024, 2);
            umma_tf32_ss(tmem_base + T::COL_S, da_lo, db_hi, idesc1, (kb == 0 && ks == 0) ? 0u : 1u);
            umma_tf32_ss(tmem_base + T::COL_S, da_hi, db_lo, idesc1, 1u);
            umma_tf32_ss(tmem_base + T::COL_S, da_hi, db_hi, idesc1, 1u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        umma_commit(&s_full_bar);
        // phase 2: O = P V, once the probabilities are in TMEM and the previous O has been read
        if (!mbar_wait(&p_ready_bar, it & 1u, abortp)) { ok = false; break; }
        if (it > 0 && !mbar_wait(&o_empty_bar, (it - 1) & 1u, abortp)) { ok = false; break; }
        tc_fence_after_sync();
        for (int kb = 0; kb < kb2; ++kb) {
          if (!mbar_wait(&split_bar[s], ph, abortp)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t b_hi = smem_u32(ring + s * T::STAGE_BYTES);
#pragma unroll
          for (int ks = 0; ks < BK / kUmmaK; ++ks) {
            const uint64_t db_hi = make_smem_desc(b_hi + ks * 1024, T::MN_CHUNK_BYTES, 512, 1);
            const uint64_t db_lo = make_smem_desc(b_hi + T::RAW2 + ks * 1024, T::MN_CHUNK_BYTES, 512, 1);
            const uint32_t col = kb * BK + ks * kUmmaK;
            umma_tf32_ts(tmem_base + T::COL_O, tmem_base + T::COL_PLO + col, db_hi, idesc2, (kb == 0 && ks == 0) ? 0u : 1u);
            umma_tf32_ts(tmem_base + T::COL_O, tmem_base + T::COL_S + col, db_lo, idesc2, 1u);
            umma_tf32_ts(tmem_base + T::COL_O, tmem_base + T::COL_S + col, db_hi, idesc2, 1u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&o_full_bar);
      }
    }
    __syncwarp();
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax + stores (one score row per lane)
    reg_alloc<T::REGS_EPI>();
    const int q = warp & 3;
    float* stage = reinterpret_cast<float*>(ring + T::RING_BYTES) + (warp - 4) * (T::EPI_STAGE_BYTES / 4);
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    uint32_t it = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++it) {
      const int b = u / p.tiles_q, m0 = (u - b * p.tiles_q) * 128;
      const int row_base = m0 + q * 32;
      if (!mbar_wait_warp(&s_full_bar, it & 1u, abortp)) { ok = false; break; }
      tc_fence_after_sync();
      float acc[TKN];
#pragma unroll
      for (int g = 0; g < TKN / 32; ++g) {
        tmem_ld_32x32(tmem_base + lane_base + T::COL_S + g * 32, acc + g * 32);
        tmem_ld_wait();
      }
      epilogue_row_op<TKN, 1>(p.s, acc, stage, row_xch, b, row_base, 0, q, 0, lane);
      // the probabilities as the A operand of the second product: raw over S, lo plane beside it
#pragma unroll
      for (int g = 0; g < TKN / 32; ++g) {
        uint32_t lo[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const uint32_t x = __float_as_uint(acc[g * 32 + j]);
          lo[j] = to_tf32_rna(acc[g * 32 + j] - __uint_as_float(x & 0xffffe000u));
        }
        tmem_st_32x32(tmem_base + lane_base + T::COL_S + g * 32, reinterpret_cast<const uint32_t*>(acc + g * 32));
        tmem_st_32x32(tmem_base + lane_base + T::COL_PLO + g * 32, lo);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready_bar);
      // `weights`, kept by the layer for its backward pass, stored while the tensor core runs the second product
      {
        StoreTarget t = {p.s.C, nullptr, nullptr, 1.0f, 0.0f, ACT_IDENTITY, p.s.ldc, p.s.vec_ok, 0};
        epilogue_store_rows<TKN>(p.s, t, acc, stage, b, static_cast<long long>(b) * p.s.strideC, row_base, 0, lane);
      }
      if (!mbar_wait_warp(&o_full_bar, it & 1u, abortp)) { ok = false; break; }
      tc_fence_after_sync();
      float o[EN];
#pragma unroll
      for (int g = 0; g < EN / 32; ++g) {
        tmem_ld_32x32(tmem_base + lane_base + T::COL_O + g * 32, o + g * 32);
        tmem_ld_wait();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&o_empty_bar);
      {
        StoreTarget t = {p.o.C, nullptr, nullptr, 1.0f, 0.0f, ACT_IDENTITY, p.o.ldc, p.o.vec_ok, p.o.omap.on};
        epilogue_store_rows<EN>(p.o, t, o, stage, b, static_cast<long long>(b) * p.o.strideC, row_base, 0, lane);
      }
    }
  } else {
    // ------------------------------------------------------------------ hi / lo split of the landed tiles
    reg_dealloc<T::REGS_SPLIT>();
    const int tid = threadIdx.x - 256;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      for (int kb = 0; kb < kb1 + kb2; ++kb) {
        if (!mbar_wait_warp(&full_bar[s], ph, abortp)) { ok = false; break; }
        if (kb < kb1) split_stage<T::RAW1, 128>(ring + s * T::STAGE_BYTES, tid, 0);
        else          split_stage<T::RAW2, 128>(ring + s * T::STAGE_BYTES, tid, 0);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&split_bar[s]);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag) atomicExch(p.error_word, 1);
}

}  // namespace snb
