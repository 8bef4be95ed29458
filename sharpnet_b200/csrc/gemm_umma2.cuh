// CTA-pair variant of the tcgen05 GEMM: two CTAs on the two SMs of a TPC compute one
// 256 x BN output tile with `tcgen05.mma.cta_group::2`.
//
// Why: with one CTA per tile the tensor core re-reads its A (128 x 8) and B (BN x 8) operand slices
// from shared memory for every instruction, and for fp32 operands that traffic plus the TMA writes
// (plus the hi/lo split in 3xTF32 mode) exceeds what one SM's shared memory can deliver -- the
// single-CTA kernel stalls at ~55 % tensor-pipe activity.  In a pair each CTA keeps its own 128 rows
// of A but only HALF of the B tile (BN/2 columns); the hardware feeds both tensor cores from the two
// halves, so per SM the B bytes that are loaded, split and read are halved.
//
// Roles per CTA (same warp layout as the single-CTA kernel): TMA producer (own A rows, own B half),
// split warps (3xTF32), epilogue warps (own 128 rows of the accumulator, which lives in this CTA's
// TMEM).  Only the even CTA issues MMAs.  Cross-CTA signalling:
//   ready[s]     (even CTA)  <- split warps of both CTAs (3xTF32) or one relay lane per CTA (TF32)
//   empty[s]     (both CTAs) <- tcgen05.commit with CTA mask 0b11 from the MMA lane
//   acc_full[b]  (both CTAs) <- tcgen05.commit with CTA mask 0b11
//   acc_empty[b] (even CTA)  <- epilogue threads of both CTAs
// Loads are plain per-CTA TMA; nothing is multicast.  Every wait is bounded.
#pragma once
#include "gemm_umma.cuh"

namespace snb {

// HYBRID_ (with SPLIT_): the second plane holds bf16 cross-term operands instead of TF32 lo values, and every 8-wide
// K slice takes one TF32 and one bf16 instruction instead of three TF32 ones (see split_stage_bf16).
template <int BN_, int BK_, bool SPLIT_, bool HYBRID_ = false>
struct Umma2Tile {
  static constexpr bool HYBRID = HYBRID_;
  static constexpr int BM = 128;                 // rows per CTA; the pair covers 256
  static constexpr int BN = BN_;                 // columns of the pair's tile
  static constexpr int BNH = BN_ / 2;            // B columns held by each CTA
  static constexpr int BK = BK_;
  static constexpr bool SPLIT = SPLIT_;
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BNH * BK * 4;
  static constexpr int RAW_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGE_BYTES = RAW_BYTES * (SPLIT ? 2 : 1);
  static constexpr int SMEM_BUDGET = 192 * 1024;
  static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;
  static constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;   // a power of two
  static constexpr int EPI_GROUPS = (BN >= 64) ? 2 : 1;
  static constexpr int EPI_THREADS = 128 * EPI_GROUPS;
  static constexpr int EPI_COLS = BN / EPI_GROUPS;
  static constexpr int SMEM_BYTES = RING_BYTES + EPI_STAGE_BYTES * 4 * EPI_GROUPS + 1024;
  static constexpr int N_SPLIT_THREADS = SPLIT ? 128 : 0;
  static constexpr int SPLIT_THREAD0 = 128 + EPI_THREADS;
  static constexpr int THREADS = 128 + EPI_THREADS + N_SPLIT_THREADS;
  static constexpr int READY_COUNT = SPLIT ? 2 * N_SPLIT_THREADS / 32 : 2;   // one arrival per split warp / relay
  static constexpr int REGS_CTRL = 56;
  static constexpr int REGS_SPLIT = 64;
  static constexpr int REGS_EPI_RAW = (65536 / 128 - REGS_CTRL - (SPLIT ? REGS_SPLIT : 0)) / EPI_GROUPS;
  static constexpr int REGS_EPI = (REGS_EPI_RAW > 232 ? 232 : REGS_EPI_RAW) / 8 * 8;
  static constexpr int KMAJ_ROW_BYTES = BK * 4;
  static constexpr int KMAJ_SBO = 8 * KMAJ_ROW_BYTES;
  static constexpr int KMAJ_LAYOUT = (BK == 32) ? 2 : 4;
  static constexpr int MNMAJ_CHUNK_BYTES = BK * 128;
  static constexpr int MNMAJ_SBO = 512;
  static constexpr int MNMAJ_LAYOUT = 1;
  static_assert(BK == 32 || BK == 16, "BK must be 16 or 32");
  static_assert(BN == 64 || BN == 128 || BN == 192 || BN == 256, "BN must be 64, 128, 192 or 256");
  static_assert(STAGES >= 2, "need at least two stages");
};

template <class T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T::THREADS, 1)
umma2_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const UmmaParams p) {
  constexpr int BM = T::BM, BN = T::BN, BNH = T::BNH, BK = T::BK, STAGES = T::STAGES;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[STAGES];    // this CTA's TMA bytes landed
  __shared__ uint64_t ready_bar[STAGES];   // (even CTA) operands of both CTAs ready for the tensor cores
  __shared__ uint64_t empty_bar[STAGES];   // MMAs that read the stage retired
  __shared__ uint64_t acc_full_bar[2];     // partial sum complete in TMEM
  __shared__ uint64_t acc_empty_bar[2];    // (even CTA) partial sum moved to registers by both CTAs
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = (rank == 0);
  uint8_t* ring = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&ready_bar[s], T::READY_COUNT);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full_bar[b], 1);
      mbar_init(&acc_empty_bar[b], 2 * T::EPI_THREADS / 32);   // one arrival per epilogue warp of either CTA
    }
    abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_holder, T::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_holder;
  volatile int* abortp = &abort_flag;
  allow_dependent_launch();   // set-up done without touching global memory: see umma_gemm_kernel
  grid_dependency_wait();

  const int pair_tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int n_tiles = p.batch * pair_tiles_m * p.tiles_n;
  const int total_tiles = p.whole_tiles + (n_tiles - p.whole_tiles) * p.splits;   // work units
  const int n_pairs = gridDim.x >> 1;
  const int pair_id = blockIdx.x >> 1;

  if (warp < 4) {
    reg_dealloc<T::REGS_CTRL>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer (both CTAs)
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += n_pairs) {
        int tile, split, kb_begin, kb_end, b, tm, tn;
        unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
        tile_coords(tile, pair_tiles_m, p.tiles_n, b, tm, tn);
        const int m0 = tm * 2 * BM + rank * BM;      // this CTA's rows of A
        const int n0 = tn * BN + rank * BNH;         // this CTA's half of B
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait_cluster(&empty_bar[s], ph ^ 1, abortp)) { ok = false; break; }
          uint8_t* a_dst = ring + s * T::STAGE_BYTES;
          uint8_t* b_dst = a_dst + T::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], T::RAW_BYTES);
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_3d(a_dst, &tmA, &full_bar[s], k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 32; ++j)
              tma_load_3d(a_dst + j * T::MNMAJ_CHUNK_BYTES, &tmA, &full_bar[s], m0 + 32 * j, k0, b);
          }
          if (!p.b_mn) {
            tma_load_3d(b_dst, &tmB, &full_bar[s], k0, n0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 32; ++j)
              tma_load_3d(b_dst + j * T::MNMAJ_CHUNK_BYTES, &tmB, &full_bar[s], n0 + 32 * j, k0, b);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    } else if (warp == 1 && lane == 0 && leader) {
      // ---------------------------------------------------------------- MMA issuer (even CTA only)
      const uint32_t idesc = make_idesc_tf32(2 * BM, BN, p.a_mn, p.b_mn);
      const uint32_t idesc16 = make_idesc_bf16(2 * BM, BN);
      const uint32_t a_step = p.a_mn ? 1024u : 32u;
      const uint32_t b_step = p.b_mn ? 1024u : 32u;
      const uint32_t a_lbo = p.a_mn ? T::MNMAJ_CHUNK_BYTES : 16u;
      const uint32_t b_lbo = p.b_mn ? T::MNMAJ_CHUNK_BYTES : 16u;
      const uint32_t a_sbo = p.a_mn ? T::MNMAJ_SBO : T::KMAJ_SBO;
      const uint32_t b_sbo = p.b_mn ? T::MNMAJ_SBO : T::KMAJ_SBO;
      const uint32_t a_lay = p.a_mn ? T::MNMAJ_LAYOUT : T::KMAJ_LAYOUT;
      const uint32_t b_lay = p.b_mn ? T::MNMAJ_LAYOUT : T::KMAJ_LAYOUT;
      int s = 0;
      uint32_t ph = 0;
      uint32_t acc_ph = 0;
      uint32_t chunk_id = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += n_pairs) {
        int tile, split, kb_begin, kb_end;
        unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
        for (int kb0 = kb_begin; kb0 < kb_end && ok; kb0 += p.chunk_kblocks, ++chunk_id) {
          const int buf = chunk_id & 1;
          if (!mbar_wait_cluster(&acc_empty_bar[buf], ((acc_ph >> buf) & 1u) ^ 1u, abortp)) { ok = false; break; }
          acc_ph ^= 1u << buf;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb1 = min(kb_end, kb0 + p.chunk_kblocks);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait_cluster(&ready_bar[s], ph, abortp)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_hi = smem_u32(ring + s * T::STAGE_BYTES);
            const uint32_t b_hi = a_hi + T::A_BYTES;
#pragma unroll
            for (int ks = 0; ks < BK / kUmmaK; ++ks) {
              const uint64_t da_hi = make_smem_desc(a_hi + ks * a_step, a_lbo, a_sbo, a_lay);
              const uint64_t db_hi = make_smem_desc(b_hi + ks * b_step, b_lbo, b_sbo, b_lay);
              const uint32_t first = (kb == kb0 && ks == 0) ? 0u : 1u;
              if (T::HYBRID) {
                const uint64_t da_16 = make_smem_desc(a_hi + T::RAW_BYTES + ks * 32u, 16u, T::KMAJ_SBO, T::KMAJ_LAYOUT);
                const uint64_t db_16 = make_smem_desc(b_hi + T::RAW_BYTES + ks * 32u, 16u, T::KMAJ_SBO, T::KMAJ_LAYOUT);
                umma_bf16_ss_pair(d_tmem, da_16, db_16, idesc16, first);      // a_lo*b_hi + a_hi*b_lo
                umma_tf32_ss_pair(d_tmem, da_hi, db_hi, idesc, 1u);
              } else if (T::SPLIT) {
                const uint64_t da_lo = make_smem_desc(a_hi + T::RAW_BYTES + ks * a_step, a_lbo, a_sbo, a_lay);
                const uint64_t db_lo = make_smem_desc(b_hi + T::RAW_BYTES + ks * b_step, b_lbo, b_sbo, b_lay);
                umma_tf32_ss_pair(d_tmem, da_lo, db_hi, idesc, first);
                umma_tf32_ss_pair(d_tmem, da_hi, db_lo, idesc, 1u);
                umma_tf32_ss_pair(d_tmem, da_hi, db_hi, idesc, 1u);
              } else {
                umma_tf32_ss_pair(d_tmem, da_hi, db_hi, idesc, first);
              }
            }
            umma_commit_pair(&empty_bar[s]);   // frees the stage in both CTAs
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
          if (ok) umma_commit_pair(&acc_full_bar[buf]);
        }
      }
    } else if (!T::SPLIT && warp == 2 && lane == 0) {
      // ---------------------------------------------------------------- relay (TF32 mode, both CTAs):
      // tells the even CTA that this CTA's tiles have landed
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += n_pairs) {
        int tile, split, kb_begin, kb_end;
        unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&full_bar[s], ph, abortp)) { ok = false; break; }
          mbar_arrive_cluster(map_to_cta(smem_u32(&ready_bar[s]), 0));
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp < 4 + 4 * T::EPI_GROUPS) {
    // ------------------------------------------------------------------ epilogue (both CTAs, own rows)
    reg_alloc<T::REGS_EPI>();
    constexpr int NC = T::EPI_COLS;
    const int q = warp & 3;
    const int col_base = ((warp - 4) >> 2) * NC;
    uint32_t acc_ph = 0;
    uint32_t chunk_id = 0;
    bool ok = true;
    for (int t = pair_id; t < total_tiles && ok; t += n_pairs) {
      int tile, split, kb_begin, kb_end, b, tm, tn;
      unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
      tile_coords(tile, pair_tiles_m, p.tiles_n, b, tm, tn);
      const int n_chunks = (kb_end - kb_begin + p.chunk_kblocks - 1) / p.chunk_kblocks;
      float* stage = reinterpret_cast<float*>(ring + T::RING_BYTES) + (warp - 4) * (T::EPI_STAGE_BYTES / 4);
      float acc[NC];
#pragma unroll
      for (int j = 0; j < NC; ++j) acc[j] = 0.0f;
      const bool c_folded = epilogue_fold_c<NC>(p, acc, stage, b, split, tm * 2 * BM + rank * BM + q * 32,
                                                tn * BN + col_base, lane);
      for (int c = 0; c < n_chunks && ok; ++c, ++chunk_id) {
        const int buf = chunk_id & 1;
        if (!mbar_wait_cluster_warp(&acc_full_bar[buf], (acc_ph >> buf) & 1u, abortp)) { ok = false; break; }
        acc_ph ^= 1u << buf;
        tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + col_base;
#pragma unroll
        for (int g = 0; g < NC / 32; ++g) {
          float v[32];
          tmem_ld_32x32(t_addr + g * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[g * 32 + j] += v[j];
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[buf]), 0));
      }
      if (!ok) break;
      epilogue_store_unit<NC>(p, p.alpha, c_folded ? 0.0f : p.beta, p.bias, acc, stage, b, n_tiles, tile, split, tm * 2 * BM, tn * BN, BN,
                              tm * 2 * BM + rank * BM + q * 32, tn * BN + col_base, lane);
    }
  } else if (T::SPLIT) {
    // ------------------------------------------------------------------ hi / lo split (both CTAs)
    reg_dealloc<T::REGS_SPLIT>();
    const int tid = threadIdx.x - T::SPLIT_THREAD0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int t = pair_id; t < total_tiles && ok; t += n_pairs) {
      int tile, split, kb_begin, kb_end;
      unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait_warp(&full_bar[s], ph, abortp)) { ok = false; break; }
        if constexpr (T::HYBRID) split_stage_bf16<T::A_BYTES, T::RAW_BYTES, T::N_SPLIT_THREADS>(ring + s * T::STAGE_BYTES, tid);
        else                     split_stage<T::RAW_BYTES, T::N_SPLIT_THREADS>(ring + s * T::STAGE_BYTES, tid, p.rewrite_hi);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ready_bar[s]), 0));
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // no CTA leaves (or frees TMEM) while its peer may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, T::TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag) atomicExch(p.error_word, 1);
}

}  // namespace snb
