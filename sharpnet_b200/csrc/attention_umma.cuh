// Scaled dot-product attention forward as ONE tcgen05 kernel (3xTF32):
//
//   weights = softmax(mask(scaling * Q K^T)),  y = weights V          per matrix of the batch
//
// for score rows that fit one tile: v_steps <= 128 and embedding_dim <= 128.  One persistent CTA per SM walks over
// work units (matrix b, block of 128 query rows).  Per unit:
//   product 1  S [128 x TKN] = Q K^T: both operands stream through the shared-memory ring in 32-deep K blocks, the
//              split warps add their lo planes, the tensor core accumulates the three TF32 products in TMEM;
//   softmax    the epilogue warps (two per score row from 64 columns up, each holding half of the row; they exchange
//              the row maximum and sum through shared memory) read S from TMEM, apply scaling, the causal overwrite
//              with -1e12 and the softmax, and write the probabilities back to TMEM as the A operand of the second
//              product -- raw over S (the tensor core truncates to TF32 itself) and lo = tf32(p - hi) beside it --
//              then store them to `weights` (the layer keeps them for its backward pass) while the tensor core works;
//   product 2  O [128 x EN] = P V with P read from TMEM (A operand in tensor memory) and V streamed through the same
//              ring as an MN-major B tile with its lo plane; the epilogue warps store O as y.
// S is double buffered in TMEM, and the ring, the split warps and the MMA lane all walk the same sequence
//   QK(0), QK(1), V(0), QK(2), V(1), ..., V(last)
// so the first product of unit u+1 runs on the tensor core while the epilogue warps are busy with the softmax of
// unit u, and the loads of later units overlap everything.  No scores buffer, no second launch, and the
// probabilities never pass through shared memory.
//
// The same kernel body, instantiated with GRAD, is the middle of the backward pass:
//
//   dScores = softmax'(scaling * dy V^T; weights),  dQ = dScores K
//
// product 1 takes dy and V in the places of Q and K, the epilogue warps apply the softmax Jacobian
// y * (g - sum_j g_j y_j) with the forward pass's probabilities read from `weights` (coalesced, through the warp's
// shared-memory tile) instead of the softmax, dScores is stored where the forward kernel stores the weights (the
// dK product reads it) and handed to product 2 through tensor memory, and K takes the place of V.
//
// Reference: ScaledDotProductAttentionLayer.ScaledDotProductAttentionForwardPropagation
// (Prod/Layers/ScaledDotProductAttentionLayer.cs:46-91) and its BackwardPropagation (:93-132).
#pragma once
#include "gemm_umma.cuh"

namespace snb {

template <int TKN_, int EN_>
struct AttnTile {
  static constexpr int TKN = TKN_;                       // score columns (v_steps padded): N of product 1, K of product 2
  static constexpr int EN = EN_;                         // embedding columns padded: K of product 1, N of product 2
  static constexpr int BK = 32;
  static constexpr int Q_BYTES = 128 * BK * 4;           // product-1 A block
  static constexpr int K_BYTES = TKN * BK * 4;           // product-1 B block
  static constexpr int RAW1 = Q_BYTES + K_BYTES;
  static constexpr int RAW2 = EN * BK * 4;               // product-2 B block: 32 rows of V
  static constexpr int STAGE1 = 2 * RAW1, STAGE2 = 2 * RAW2;   // raw tiles + lo planes
  static constexpr int STAGE_BYTES = STAGE1 > STAGE2 ? STAGE1 : STAGE2;
  static constexpr int G = TKN >= 64 ? 2 : 1;            // epilogue warps per score row
  static constexpr int NC = TKN / G;                     // score columns per epilogue warp
  static constexpr int OG = (G == 2 && EN >= 64) ? 2 : 1;   // warp groups that share the columns of O
  static constexpr int NCO = EN / OG;
  static constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;
  static constexpr int EPI_BYTES = 4 * G * EPI_STAGE_BYTES;
  static constexpr int STAGES_RAW = (225 * 1024 - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = RING_BYTES + EPI_BYTES + 1024;
  static constexpr int SPLIT_THREAD0 = 128 + 128 * G;
  static constexpr int THREADS = SPLIT_THREAD0 + 128;    // 4 control warps, 4 G epilogue warps, 4 split warps
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S0 = 0, COL_PLO = 2 * TKN, COL_O = 3 * TKN;   // TMEM columns; S buffer b at b * TKN
  static constexpr int REGS_CTRL = 72, REGS_SPLIT = 64;
  static constexpr int REGS_LAUNCH = (65536 / THREADS) / 8 * 8;   // what the CTA is launched with, per thread
  static constexpr int REGS_EPI_RAW = (THREADS / 128 * REGS_LAUNCH - REGS_CTRL - REGS_SPLIT) / G;
  static constexpr int REGS_EPI = (REGS_EPI_RAW > 232 ? 232 : REGS_EPI_RAW) / 8 * 8;
  static_assert(REGS_CTRL + REGS_SPLIT + G * REGS_EPI <= THREADS / 128 * REGS_LAUNCH, "register shares exceed the CTA's pool");
  static constexpr int MN_CHUNK_BYTES = BK * 128;
  static_assert(TKN == 32 || TKN == 64 || TKN == 128, "score tile 32, 64 or 128 wide");
  static_assert(EN == 32 || EN == 64 || EN == 128, "embedding tile 32, 64 or 128 wide");
  static_assert(STAGES >= 2, "need two stages");
  static_assert(3 * TKN + EN <= 512, "TMEM columns");
  static_assert(SMEM_BYTES <= 227 * 1024 - 512, "shared memory");
};

struct AttnParams {
  int batch, q_steps, v_steps, embedding_dim;
  int tiles_q;            // blocks of 128 query rows per matrix
  UmmaParams s;           // placement of `weights` [batch, q_steps, v_steps], scaling in alpha, causal, row_op
  UmmaParams o;           // placement of y [batch, q_steps, embedding_dim] (possibly mapped)
  int* error_word;
};

template <class T, bool GRAD>
__device__ __forceinline__ void attn_core(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                          const AttnParams& p) {
  constexpr int TKN = T::TKN, EN = T::EN, BK = T::BK, STAGES = T::STAGES, G = T::G, NC = T::NC;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[STAGES], split_bar[STAGES], empty_bar[STAGES];
  __shared__ uint64_t s_full_bar[2], p_ready_bar, o_full_bar, o_empty_bar;
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;
  __shared__ float row_xch[2 * 128];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* ring = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  if (threadIdx.x == 0) SNB_STAMP(p.s, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&split_bar[s], 4);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&s_full_bar[0], 1);
    mbar_init(&s_full_bar[1], 1);
    mbar_init(&p_ready_bar, 4 * G);
    mbar_init(&o_full_bar, 1);
    mbar_init(&o_empty_bar, 4 * T::OG);
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
  if (threadIdx.x == 0) SNB_STAMP(p.s, 2);

  const int units = p.batch * p.tiles_q;
  const int n_local = blockIdx.x < units ? (units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;   // this CTA's units
  const int kb1 = (p.embedding_dim + BK - 1) / BK;       // K blocks of product 1
  const int kb2 = (p.v_steps + BK - 1) / BK;             // K blocks of product 2
  // Step i of the common sequence: QK(i) if i < n_local, then V(i - 1) if i > 0.

  if (warp < 4) {
    reg_dealloc<T::REGS_CTRL>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int i = 0; i <= n_local && ok; ++i) {
        if (i < n_local) {
          const int u = blockIdx.x + i * gridDim.x;
          const int b = u / p.tiles_q, m0 = (u - b * p.tiles_q) * 128;
          for (int kb = 0; kb < kb1; ++kb) {
            if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) { ok = false; break; }
            uint8_t* dst = ring + s * T::STAGE_BYTES;
            if (i == 0 && kb == 0) SNB_STAMP(p.s, 3);
            mbar_arrive_expect_tx(&full_bar[s], T::RAW1);
            tma_load_3d(dst, &tmQ, &full_bar[s], kb * BK, m0, b);
            tma_load_3d(dst + T::Q_BYTES, &tmK, &full_bar[s], kb * BK, 0, b);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
        if (i > 0 && ok) {
          const int u = blockIdx.x + (i - 1) * gridDim.x;
          const int b = u / p.tiles_q;
          for (int kb = 0; kb < kb2; ++kb) {
            if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) { ok = false; break; }
            uint8_t* dst = ring + s * T::STAGE_BYTES;
            mbar_arrive_expect_tx(&full_bar[s], T::RAW2);
#pragma unroll
            for (int j = 0; j < EN / 32; ++j)
              tma_load_3d(dst + j * T::MN_CHUNK_BYTES, &tmV, &full_bar[s], 32 * j, kb * BK, b);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      const uint32_t idesc1 = make_idesc_tf32(128, TKN, 0, 0);
      const uint32_t idesc2 = make_idesc_tf32(128, EN, 0, 1);
      const uint64_t kdesc = make_smem_desc(0, 16, 1024, 2);                       // K-major, 128-byte swizzle
      const uint64_t vdesc = make_smem_desc(0, T::MN_CHUNK_BYTES, 512, 1);         // MN-major, 32-byte atoms
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int i = 0; i <= n_local && ok; ++i) {
        if (i < n_local) {
          // product 1 of unit i into S buffer i & 1.  The buffer is free: the product that read the probabilities of
          // unit i - 2 from these columns was issued before, and the tensor core runs one thread's instructions in order.
          const uint32_t d_s = tmem_base + (i & 1) * TKN;
          for (int kb = 0; kb < kb1; ++kb) {
            if (!mbar_wait(&split_bar[s], ph, abortp)) { ok = false; break; }
            if (kb == 0) SNB_STAMP(p.s, i == 0 ? 5 : 24);
            tc_fence_after_sync();
            const uint32_t a_hi = smem_u32(ring + s * T::STAGE_BYTES);
            const uint64_t da0 = kdesc + ((a_hi & 0x3ffffu) >> 4), db0 = kdesc + (((a_hi + T::Q_BYTES) & 0x3ffffu) >> 4);
#pragma unroll
            for (int ks = 0; ks < BK / kUmmaK; ++ks) {
              const uint64_t da_hi = da0 + ks * 2, db_hi = db0 + ks * 2;          // 32 bytes per K slice
              umma_tf32_ss(d_s, da_hi + (T::RAW1 >> 4), db_hi, idesc1, (kb == 0 && ks == 0) ? 0u : 1u);
              umma_tf32_ss(d_s, da_hi, db_hi + (T::RAW1 >> 4), idesc1, 1u);
              umma_tf32_ss(d_s, da_hi, db_hi, idesc1, 1u);
            }
            umma_commit(&empty_bar[s]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
          if (!ok) break;
          umma_commit(&s_full_bar[i & 1]);
          SNB_STAMP(p.s, i == 0 ? 6 : 25);
        }
        if (i > 0) {
          // product 2 of unit j = i - 1, once its probabilities are in TMEM and the previous O has been read
          const int j = i - 1;
          if (!mbar_wait(&p_ready_bar, j & 1u, abortp)) { ok = false; break; }
          if (j > 0 && !mbar_wait(&o_empty_bar, (j - 1) & 1u, abortp)) { ok = false; break; }
          SNB_STAMP(p.s, j == 0 ? 20 : 26);
          tc_fence_after_sync();
          const uint32_t a_hi_t = tmem_base + (j & 1) * TKN, a_lo_t = tmem_base + T::COL_PLO;
          for (int kb = 0; kb < kb2; ++kb) {
            if (!mbar_wait(&split_bar[s], ph, abortp)) { ok = false; break; }
            tc_fence_after_sync();
            const uint64_t db0 = vdesc + ((smem_u32(ring + s * T::STAGE_BYTES) & 0x3ffffu) >> 4);
#pragma unroll
            for (int ks = 0; ks < BK / kUmmaK; ++ks) {
              const uint64_t db_hi = db0 + ks * 64;                                // 1024 bytes per K slice
              const uint32_t col = kb * BK + ks * kUmmaK;
              umma_tf32_ts(tmem_base + T::COL_O, a_lo_t + col, db_hi, idesc2, (kb == 0 && ks == 0) ? 0u : 1u);
              umma_tf32_ts(tmem_base + T::COL_O, a_hi_t + col, db_hi + (T::RAW2 >> 4), idesc2, 1u);
              umma_tf32_ts(tmem_base + T::COL_O, a_hi_t + col, db_hi, idesc2, 1u);
            }
            umma_commit(&empty_bar[s]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
          if (ok) umma_commit(&o_full_bar);
          SNB_STAMP(p.s, j == 0 ? 21 : 27);
        }
      }
    }
    __syncwarp();
  } else if (warp < 4 + 4 * G) {
    // ------------------------------------------------------------------ softmax + stores
    reg_alloc<T::REGS_EPI>();
    const int q = warp & 3;                      // TMEM lane quarter: score rows q * 32 .. + 31 of the block
    const int grp = (warp - 4) >> 2;             // which part of the columns this warp holds
    const int col_base = grp * NC;
    float* stage = reinterpret_cast<float*>(ring + T::RING_BYTES) + (warp - 4) * (T::EPI_STAGE_BYTES / 4);
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_local && ok; ++it) {
      const int u = blockIdx.x + it * gridDim.x;
      const int b = u / p.tiles_q, m0 = (u - b * p.tiles_q) * 128;
      const int row_base = m0 + q * 32;
      const uint32_t s_col = tmem_base + lane_base + (it & 1) * TKN + col_base;
      ok = mbar_wait_warp(&s_full_bar[it & 1], (it >> 1) & 1u, abortp);
      if (warp == 4 && lane == 0) SNB_STAMP(p.s, it == 0 ? 7 : 28);
      if (G == 2) ok = row_pair_all(row_xch, q, grp, lane, ok);   // both warps of a row go on, or neither
      if (!ok) break;
      tc_fence_after_sync();
      // The row is walked in blocks of 32 columns with ROLLED loops that re-read the block from TMEM each time: fully
      // unrolled over the whole row, this code is several thousand instructions that every warp runs once per unit,
      // and the warps then wait for instruction fetches more than for anything else (measured: 16 % of the
      // instruction-cache requests missed, "no instruction" the top stall reason).  TMEM reads are cheap.
      const float alpha = p.s.alpha;
      if constexpr (GRAD) {
        // softmax Jacobian: dS = y * (g - sum_j g_j y_j), g = alpha * S, y = the forward pass's probabilities
        // (0 in masked columns, so the mask needs no second application: Prod/GPU/GpuTensor.cs:445-490)
        const float* yrow = p.s.aux + static_cast<long long>(b) * p.s.strideC + static_cast<long long>(row_base) * p.s.ldc;
        const int rows_valid = p.s.M - row_base;
        // The lane's NC probabilities stay in registers between the two passes (both loops unrolled: NC / 32 is 1 or
        // 2 with two warps per row, and a rolled loop would index the array dynamically).
        float d4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        float ykeep[NC];
#pragma unroll
        for (int g = 0; g < NC / 32; ++g) {
          float v[32], y[32];
          tmem_ld_32x32(s_col + g * 32, v);
          const int c0 = col_base + g * 32;
          epilogue_load_block(yrow + c0, p.s.ldc, rows_valid, p.s.N - c0, stage, lane, y);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            d4[j & 3] = fmaf(alpha * v[j], y[j], d4[j & 3]);
            ykeep[g * 32 + j] = y[j];
          }
        }
        float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
        if (G == 2) {
          const float other = row_pair_exchange(row_xch, q, grp, lane, dot);
          dot = grp == 0 ? dot + other : other + dot;   // same order in both warps
        }
#pragma unroll
        for (int g = 0; g < NC / 32; ++g) {
          float v[32];
          uint32_t lo[32];
          tmem_ld_32x32(s_col + g * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            v[j] = ykeep[g * 32 + j] * (alpha * v[j] - dot);
            lo[j] = to_tf32_rna(v[j] - __uint_as_float(__float_as_uint(v[j]) & 0xffffe000u));
          }
          tmem_st_32x32(s_col + g * 32, reinterpret_cast<const uint32_t*>(v));
          tmem_st_32x32(tmem_base + lane_base + T::COL_PLO + col_base + g * 32, lo);
        }
      } else {
      const int row = row_base + lane;
      const int limit = p.s.causal ? row : 0x7fffffff;          // columns > limit are masked
      // pass 1: row maximum of mask(alpha * S)
      float mx = -3.402823466e38f;
#pragma unroll 1
      for (int g = 0; g < NC / 32; ++g) {
        float v[32];
        tmem_ld_32x32(s_col + g * 32, v);
        tmem_ld_wait();
        const int c0 = col_base + g * 32;
        float m4[4] = {-3.402823466e38f, -3.402823466e38f, -3.402823466e38f, -3.402823466e38f};
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float x = (c0 + j > limit) ? -1e12f : alpha * v[j];
          x = (c0 + j < p.s.N) ? x : -3.402823466e38f;
          m4[j & 3] = fmaxf(m4[j & 3], x);
        }
        mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
      }
      if (G == 2) mx = fmaxf(mx, row_pair_exchange(row_xch, q, grp, lane, mx));
      if (warp == 4 && lane == 0 && it == 0) SNB_STAMP(p.s, 13);
      // pass 2: e = exp(x - max) written back over S, and the row sum
      const float c = mx * 1.4426950408889634f;
      float sum = 0.0f;
#pragma unroll 1
      for (int g = 0; g < NC / 32; ++g) {
        float v[32];
        tmem_ld_32x32(s_col + g * 32, v);
        tmem_ld_wait();
        const int c0 = col_base + g * 32;
        float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float x = (c0 + j > limit) ? -1e12f : alpha * v[j];
          float e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(x, 1.4426950408889634f, -c)));
          e = (c0 + j < p.s.N) ? e : 0.0f;
          v[j] = e;
          s4[j & 3] += e;
        }
        sum += (s4[0] + s4[1]) + (s4[2] + s4[3]);
        tmem_st_32x32(s_col + g * 32, reinterpret_cast<const uint32_t*>(v));
      }
      tmem_st_wait();
      if (G == 2) {
        const float other = row_pair_exchange(row_xch, q, grp, lane, sum);
        sum = grp == 0 ? sum + other : other + sum;   // same order in both warps: identical results
      }
      const float inv = 1.0f / sum;
      if (warp == 4 && lane == 0 && it == 0) SNB_STAMP(p.s, 14);
      // pass 3: the probabilities as the A operand of the second product: p over S (the tensor core truncates to
      // TF32 itself), lo = tf32(p - hi) beside it
#pragma unroll 1
      for (int g = 0; g < NC / 32; ++g) {
        float v[32];
        uint32_t lo[32];
        tmem_ld_32x32(s_col + g * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          v[j] *= inv;
          lo[j] = to_tf32_rna(v[j] - __uint_as_float(__float_as_uint(v[j]) & 0xffffe000u));
        }
        tmem_st_32x32(s_col + g * 32, reinterpret_cast<const uint32_t*>(v));
        tmem_st_32x32(tmem_base + lane_base + T::COL_PLO + col_base + g * 32, lo);
      }
      }   // !GRAD
      if (warp == 4 && lane == 0 && it == 0) SNB_STAMP(p.s, 15);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready_bar);
      if (warp == 4 && lane == 0) SNB_STAMP(p.s, it == 0 ? 8 : 29);
      // pass 4: `weights`, kept by the layer for its backward pass, read back from TMEM and stored while the tensor
      // core runs the second product
      {
        const StoreTarget t = {p.s.C, nullptr, nullptr, 1.0f, 0.0f, ACT_IDENTITY, p.s.ldc, p.s.vec_ok, 0};
#pragma unroll 1
        for (int g = 0; g < NC / 32; ++g) {
          float v[32];
          tmem_ld_32x32(s_col + g * 32, v);
          tmem_ld_wait();
          epilogue_store_rows<32>(p.s, t, v, stage, b, static_cast<long long>(b) * p.s.strideC, row_base, col_base + g * 32, lane);
        }
      }
      if (warp == 4 && lane == 0) SNB_STAMP(p.s, it == 0 ? 9 : 30);
      // every warp waits for the second product: only then may the next unit's probabilities be written
      tc_fence_before_sync();
      if (!mbar_wait_warp(&o_full_bar, it & 1u, abortp)) { ok = false; break; }
      if (warp == 4 && lane == 0) SNB_STAMP(p.s, it == 0 ? 22 : 31);
      if (grp < T::OG) {
        tc_fence_after_sync();
        const StoreTarget t = {p.o.C, nullptr, nullptr, 1.0f, 0.0f, ACT_IDENTITY, p.o.ldc, p.o.vec_ok, p.o.omap.on};
#pragma unroll 1
        for (int g = 0; g < T::NCO / 32; ++g) {
          float o[32];
          tmem_ld_32x32(tmem_base + lane_base + T::COL_O + grp * T::NCO + g * 32, o);
          tmem_ld_wait();
          if (g == T::NCO / 32 - 1) {          // O is in registers: the next second product may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_empty_bar);
          }
          epilogue_store_rows<32>(p.o, t, o, stage, b, static_cast<long long>(b) * p.o.strideC, row_base,
                                  grp * T::NCO + g * 32, lane);
        }
      }
      if (warp == 4 && lane == 0) SNB_STAMP(p.s, it == 0 ? 10 : 23);
    }
  } else {
    // ------------------------------------------------------------------ hi / lo split of the landed tiles
    reg_dealloc<T::REGS_SPLIT>();
    const int tid = threadIdx.x - T::SPLIT_THREAD0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int i = 0; i <= n_local && ok; ++i) {
      const int n1 = i < n_local ? kb1 : 0, n2 = i > 0 ? kb2 : 0;
      for (int kb = 0; kb < n1 + n2; ++kb) {
        if (!mbar_wait_warp(&full_bar[s], ph, abortp)) { ok = false; break; }
        if (kb < n1) split_stage<T::RAW1, 128>(ring + s * T::STAGE_BYTES, tid, 0);
        else         split_stage<T::RAW2, 128>(ring + s * T::STAGE_BYTES, tid, 0);
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
  if (threadIdx.x == 0) SNB_STAMP(p.s, 12);
}

template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  attn_core<T, false>(tmQ, tmK, tmV, p);
}

// dScores and dQ of the backward pass: tmQ describes dy, tmK describes V, tmV describes K (see the header comment).
template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  attn_core<T, true>(tmQ, tmK, tmV, p);
}

}  // namespace snb
