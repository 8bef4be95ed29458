// tcgen05 / TMEM GEMM for sm_100a, fp32 in and out.
//
//   C[b] = epi(alpha * op(A[b]) * op(B[b]) + beta * C[b])
//
// One persistent CTA per SM walks over 128 x BN output tiles.  Warp roles:
//   warp 0         TMA producer: fp32 tiles of A and B -> shared memory ring (swizzled)
//   warp 1         owns TMEM; one lane issues tcgen05.mma (kind::tf32) into a TMEM accumulator
//   warps 4..7/11  epilogue: TMEM partial sums -> fp32 registers -> alpha/beta/bias/activation -> global
//   last 4 warps   (3xTF32 only) split every fp32 operand tile into hi + lo TF32 planes
// The TMEM accumulator is double buffered, so draining one partial sum (or the epilogue of tile i)
// overlaps the tensor-core work on the next.
//
// Transposes never move data: an operand whose contraction dimension is contiguous in memory is
// loaded as a K-major tile, the other kind as an MN-major tile, and the tcgen05 descriptors name
// the layout.  Both are fetched by plain (non-multicast) TMA.
//
// 3xTF32: a = a_hi + a_lo with a_hi = tf32(a), a_lo = tf32(a - a_hi); the product is
// a_lo*b_hi + a_hi*b_lo + a_hi*b_hi accumulated in fp32, which recovers fp32-level accuracy
// from TF32 tensor cores.  In TF32 mode the raw fp32 tiles feed the tensor core directly.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace snb {

constexpr int kUmmaBM = 128;
constexpr int kUmmaK = 8;  // K extent of one kind::tf32 instruction

// GROUPS_ = 0 picks the number of epilogue warp groups from the tile width; the row-operation kernels ask for 2 so
// that two warps share every row (see epilogue_row_op).
// TS_ (3xTF32, BN <= 128): the A operand goes to the tensor core from tensor memory instead of shared memory.  The
// split warps, which read every landed A tile anyway, write its hi and lo planes into TMEM (64 columns per stage,
// behind the two accumulators), so the 3 x BK/8 instructions of a K block read only B from shared memory: per K
// block and SM the shared-memory traffic of a 128 x 32 tile falls from 120 KB to 56 KB, of a 128 x 128 tile from
// 192 KB to 128 KB -- and shared-memory bandwidth is what bounds this kernel.
// SWLOAD_: operands that TMA cannot load (a base that is only 4-byte aligned, a row pitch that is not a multiple of
// 16 bytes -- SharpNet slices tensors at float granularity) are brought in by four loader warps instead, which
// build in shared memory exactly the swizzled tiles TMA would have delivered (see sw_load_tile); everything after
// the `full` barrier is unchanged.
template <int BN_, int BK_, bool SPLIT_, int GROUPS_ = 0, bool TS_ = false, bool SWLOAD_ = false>
struct UmmaTile {
  static constexpr bool SWLOAD = SWLOAD_;
  static constexpr int N_LOAD_THREADS = SWLOAD_ ? 128 : 0;
  static constexpr int REGS_LOAD = 80;
  static constexpr int BM = kUmmaBM;
  static constexpr int BN = BN_;
  static constexpr int BK = BK_;
  static constexpr bool SPLIT = SPLIT_;
  static constexpr bool TS = TS_;
  static constexpr int A_BYTES = BM * BK * 4;
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int RAW_BYTES = A_BYTES + B_BYTES;               // what TMA delivers per stage
  // + the lo planes: of A and B behind the raw tiles, or (TS) of B alone
  static constexpr int STAGE_BYTES = TS ? RAW_BYTES + B_BYTES : RAW_BYTES * (SPLIT ? 2 : 1);
  static constexpr int B_LO_OFFSET = TS ? B_BYTES : RAW_BYTES;      // from the raw B tile to its lo plane
  static constexpr int SMEM_BUDGET = 196 * 1024;
  static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int TS_A_COLS = 2 * BK;                          // TMEM columns of one stage's A: hi plane, lo plane
  static constexpr int STAGES_TMEM = TS ? (512 - 2 * BN) / TS_A_COLS : 8;
  static constexpr int STAGES_CAP = STAGES_TMEM > 8 ? 8 : STAGES_TMEM;
  static constexpr int STAGES = STAGES_RAW > STAGES_CAP ? STAGES_CAP : STAGES_RAW;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int EPI_STAGE_BYTES = 32 * 32 * 4;              // one 32 x 32 fp32 block per epilogue warp
  static constexpr int TMEM_COLS = TS ? 512 : (2 * BN < 32 ? 32 : 2 * BN);   // two accumulators (+ A stages); power of two
  static constexpr int TS_A_COL0 = 2 * BN;                          // first TMEM column of the A stages
  // Warps are grouped in fours so that setmaxnreg can move registers between the roles:
  //   group 0: TMA producer, MMA issuer (two idle warps); then the epilogue groups; then the split group.
  static constexpr int EPI_GROUPS = GROUPS_ ? GROUPS_ : ((BN >= 64) ? 2 : 1);   // each epilogue warp owns <= 128 columns
  static constexpr int EPI_THREADS = 128 * EPI_GROUPS;
  static constexpr int EPI_COLS = BN / EPI_GROUPS;                  // columns per epilogue warp
  static constexpr int SMEM_BYTES = RING_BYTES + EPI_STAGE_BYTES * 4 * EPI_GROUPS + 1024;  // + 1 KB alignment slack
  static constexpr int N_SPLIT_THREADS = SPLIT ? 128 : 0;
  static constexpr int SPLIT_THREAD0 = 128 + EPI_THREADS;
  static constexpr int LOAD_THREAD0 = 128 + EPI_THREADS + N_SPLIT_THREADS;
  static constexpr int THREADS = 128 + EPI_THREADS + N_SPLIT_THREADS + N_LOAD_THREADS;
  static constexpr int REGS_CTRL = SWLOAD ? 56 : 72;
  static constexpr int REGS_SPLIT = TS ? 112 : 64;                  // TS: a whole A row and its lo plane in registers
  // setmaxnreg only moves registers inside what the CTA was launched with: THREADS x (the per-thread count the
  // kernel is compiled for, 65536 / THREADS rounded down to a multiple of 8).  A group that asks for more than the
  // other groups have given back waits for ever, so the shares must add up to at most that pool.
  static constexpr int REGS_LAUNCH = (65536 / THREADS) / 8 * 8 > 255 ? 248 : (65536 / THREADS) / 8 * 8;
  static constexpr int REG_POOL_PER_128 = THREADS / 128 * REGS_LAUNCH;
  static constexpr int REGS_EPI_RAW =
      (REG_POOL_PER_128 - REGS_CTRL - (SPLIT ? REGS_SPLIT : 0) - (SWLOAD ? REGS_LOAD : 0)) / EPI_GROUPS;
  static constexpr int REGS_EPI = (REGS_EPI_RAW > 232 ? 232 : REGS_EPI_RAW) / 8 * 8;
  static_assert(REGS_CTRL + EPI_GROUPS * REGS_EPI + (SPLIT ? REGS_SPLIT : 0) + (SWLOAD ? REGS_LOAD : 0) <= REG_POOL_PER_128,
                "register shares exceed what the CTA is launched with");
  static_assert(REGS_CTRL <= REGS_LAUNCH && REGS_SPLIT <= REGS_LAUNCH && REGS_LOAD <= REGS_LAUNCH,
                "setmaxnreg.dec must not raise the count");
  // K-major tiles: one row = BK fp32.  128-byte swizzle for BK = 32, 64-byte for BK = 16.
  static constexpr int KMAJ_ROW_BYTES = BK * 4;
  static constexpr int KMAJ_SBO = 8 * KMAJ_ROW_BYTES;
  static constexpr int KMAJ_LAYOUT = (BK == 32) ? 2 : 4;
  // MN-major tiles: chunks of 32 fp32 (128 B) along M/N, BK rows each.  32-bit MN-major operands
  // use the 128-byte swizzle with 32-byte atoms (descriptor layout 1, TMA SWIZZLE_128B_ATOM_32B):
  // the pattern repeats every 4 rows, so the stride between K groups is 4 x 128 B.
  static constexpr int MNMAJ_CHUNK_BYTES = BK * 128;
  static constexpr int MNMAJ_SBO = 512;
  static constexpr int MNMAJ_LAYOUT = 1;
  static_assert(BK == 32 || BK == 16, "BK must be 16 or 32");
  static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "BN must be 32, 64, 128 or 256");
  static_assert(STAGES >= 2, "need at least two stages");
  static_assert(EPI_COLS % 32 == 0 && EPI_COLS <= 128, "an epilogue warp keeps at most 128 columns in registers");
  static_assert(!TS || (SPLIT && BK == 32 && BN <= 128), "A from tensor memory: 3xTF32, 32-deep K blocks, BN <= 128");
  static_assert(!SWLOAD || (BK == 32 && BN <= 128 && !TS), "loader warps: 32-deep K blocks, tiles up to 128 wide");
};

struct UmmaParams {
  int M, N, K, batch;
  int tiles_m, tiles_n, k_blocks;
  int chunk_kblocks;  // k-blocks accumulated inside the tensor core before the sum moves to registers
  int a_mn, b_mn;     // 1 = operand tile is MN-major (A stored [K x M] / B stored [K x N])
  int ldc;
  long long strideC;
  float* C;
  float* Z;
  const float* bias;
  float alpha, beta;
  int act;
  float act_alpha;  // coefficient of ELU / LeakyRelu
  int rewrite_hi;   // 3xTF32: store the rounded hi plane back over the raw tile
  int vec_ok;       // C (and Z, bias) rows are 16-byte aligned
  int* error_word;  // set to 1 when a pipeline wait timed out
  // split-K.  The first `whole_tiles` tiles (in tile_coords order) are computed whole; each of the
  // remaining "tail" tiles is cut into `splits` work units of kb_per_split k-blocks that store raw partial
  // sums to the workspace, and a second kernel combines them.  Two workspace layouts:
  //   dense (partial_tiled = 0, whole_tiles = 0): split s writes a [batch, M, N] matrix at partial + s * partial_stride;
  //   tiled (partial_tiled = 1): unit (tail tile j, split s) writes its tile, row pitch BN, at
  //                              partial + (s * tail + j) * partial_stride.
  int splits;
  int kb_per_split;
  int whole_tiles;
  int partial_tiled;
  float* partial;
  long long partial_stride;
  // row operation on alpha * acc before the store (single-CTA kernel, one tile column, BN <= 128): see RowOp
  int row_op;
  int causal;
  const float* aux;
  OutMap omap;   // placement of C / Z when not dense (see OutMap)
  // K cut inside a thread-block cluster (the CLUSTER instantiations): CTA r of a cluster of `cluster` computes K
  // part r of the cluster's tile, and the parts are summed through distributed shared memory (no workspace, no
  // second kernel).  store_t = 1: the kernel ran the transposed problem and stores tile element (row, col) at
  // C[col * ldc + row], so C, Z and ldc are those of the caller's matrix and bias runs along the tile's rows.
  int cluster;
  int store_t;
  // Two products of the same shape in one launch (the GROUPED instantiation): matrices [0, group_batch) of the
  // batch are problem 1 (tmA, tmB, C), matrices [group_batch, batch) problem 2 (tmA2, tmB2), whose results land
  // c_shift floats away from where C + b * strideC (or the mapped placement of matrix b) would put them.
  int group_batch;
  long long c_shift;
  // operands as plain pointers, for the kernels whose loader warps replace TMA
  const float* A;
  const float* B;
  int lda, ldb;
  long long strideA, strideB;
#ifdef SNB_TRACE
  unsigned long long* trace;   // development builds only: %globaltimer stamps of CTA 0 (see SNB_STAMP)
#endif
};

// Development builds (-DSNB_TRACE) record where the time of one CTA goes; product builds compile none of it.
#ifdef SNB_TRACE
#define SNB_STAMP(p, slot) do { if ((p).trace != nullptr && blockIdx.x == 0) (p).trace[slot] = globaltimer_ns(); } while (0)
#else
#define SNB_STAMP(p, slot) do { } while (0)
#endif

#ifdef SNB_SLOW_ISSUE
constexpr bool kSlowIssue = true;    // development builds: every descriptor rebuilt from scratch (A/B measurements)
#else
constexpr bool kSlowIssue = false;
#endif

// Work unit u of a launch over n_tiles output tiles: which tile, which K range, and (split >= 0) which
// partial result it produces.
__device__ __forceinline__ void unit_decode(const UmmaParams& p, int n_tiles, int u, int& tile, int& split,
                                            int& kb_begin, int& kb_end) {
  if (p.cluster > 1) {      // consecutive CTAs (one cluster) share a tile
    tile = u / p.cluster; split = u - tile * p.cluster;
    kb_begin = split * p.kb_per_split;
    kb_end = min(p.k_blocks, kb_begin + p.kb_per_split);
  } else if (u < p.whole_tiles) {
    tile = u; split = -1; kb_begin = 0; kb_end = p.k_blocks;
  } else {
    const int tail = n_tiles - p.whole_tiles;
    const int v = u - p.whole_tiles;
    split = v / tail;
    tile = p.whole_tiles + (v - split * tail);
    kb_begin = split * p.kb_per_split;
    kb_end = min(p.k_blocks, kb_begin + p.kb_per_split);
  }
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& b, int& tm, int& tn) {
  // Walk tiles in bands of 8 tile-rows so that CTAs running at the same time share A and B
  // tiles through L2.
  const int per_batch = tiles_m * tiles_n;
  b = t / per_batch;
  int r = t - b * per_batch;
  const int band = 8 * tiles_n;
  const int g = r / band;
  const int first_m = g * 8;
  const int rows = min(tiles_m - first_m, 8);
  r -= g * band;
  tm = first_m + r % rows;
  tn = r / rows;
}

__device__ __forceinline__ uint32_t to_tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// One 32 x 32 block of the store phase, rows 16-byte aligned: every lane moves one float4 of 8 rows.
// HEAVY selects the transcendental activations (Swish, Tanh, Sigmoid).  Their inlined code is long, and
// fully unrolled it outgrows the instruction cache (the fetch misses cost more than the stores), so that
// variant keeps the row loop rolled; Identity and Relu are a select and stay unrolled so that the
// loads of beta*C overlap.  MAPPED places the result through p.omap (integer divisions per row: also rolled,
// and kept out of the plain variants for the same reason).
// Where and how one work unit's values are stored: the kernel's own epilogue parameters, or the workspace for
// raw partial sums.  (A handful of fields instead of a copy of UmmaParams keeps the epilogue's register count.)
struct StoreTarget {
  float* C;
  float* Z;
  const float* bias;
  float alpha, beta;
  int act, ldc, vec_ok, mapped;
  float act_alpha;
};

template <bool HEAVY, bool MAPPED>
__device__ __forceinline__ void epilogue_store_block_vec(const UmmaParams& p, const StoreTarget& t, const float* stage,
                                                         int b, long long tile_off, int row_base, int col0, int lane) {
  const int c4 = lane & 7;
  const int col = col0 + 4 * c4;
  float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (t.bias) bv = __ldg(reinterpret_cast<const float4*>(t.bias + col));
  const bool relu = t.act == ACT_RELU;
  long long col_part = col;
  if (MAPPED) {
    col_part = static_cast<long long>(col / p.omap.d) * p.omap.s_co + (col % p.omap.d);
    tile_off = static_cast<long long>(b / p.omap.H) * p.omap.s_io + static_cast<long long>(b % p.omap.H) * p.omap.s_ii;
  }
#pragma unroll((HEAVY || MAPPED) ? 1 : 8)
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3);
    const int row = row_base + r;
    if (row < p.M) {
      const float4 a4 = *reinterpret_cast<const float4*>(stage + r * 32 + ((c4 ^ (r & 7)) << 2));
      long long off;
      if (MAPPED)
        off = tile_off + static_cast<long long>(row / p.omap.T) * p.omap.s_ro +
              static_cast<long long>(row % p.omap.T) * p.omap.s_ri + col_part;
      else
        off = tile_off + static_cast<long long>(row) * t.ldc + col;
      float4 o;
      o.x = t.alpha * a4.x; o.y = t.alpha * a4.y; o.z = t.alpha * a4.z; o.w = t.alpha * a4.w;
      if (t.beta != 0.0f) {
        const float4 cin = *reinterpret_cast<const float4*>(t.C + off);
        o.x = fmaf(t.beta, cin.x, o.x);
        o.y = fmaf(t.beta, cin.y, o.y);
        o.z = fmaf(t.beta, cin.z, o.z);
        o.w = fmaf(t.beta, cin.w, o.w);
      }
      o.x += bv.x; o.y += bv.y; o.z += bv.z; o.w += bv.w;
      if (t.Z) *reinterpret_cast<float4*>(t.Z + off) = o;
      if (HEAVY) {
        o.x = act_forward(t.act, o.x, t.act_alpha);
        o.y = act_forward(t.act, o.y, t.act_alpha);
        o.z = act_forward(t.act, o.z, t.act_alpha);
        o.w = act_forward(t.act, o.w, t.act_alpha);
      } else {
        o.x = relu ? fmaxf(o.x, 0.0f) : o.x;
        o.y = relu ? fmaxf(o.y, 0.0f) : o.y;
        o.z = relu ? fmaxf(o.z, 0.0f) : o.z;
        o.w = relu ? fmaxf(o.w, 0.0f) : o.w;
      }
      *reinterpret_cast<float4*>(t.C + off) = o;
    }
  }
}

// Operand split of the TF32 + bf16 scheme: x = hi + lo with hi = x truncated to TF32 (what the tensor core reads from
// the raw tile).  The two cross terms a_lo*b_hi + a_hi*b_lo are 2^-11 of the product, so bf16 carries them: for every
// 8-wide K slice the second plane holds 16 bf16 values per row -- [lo(8) | hi(8)] for A, [hi(8) | lo(8)] for B --
// and ONE bf16 instruction of K = 16 over that slice yields both cross terms.  A 32-deep K block is 4 such slices
// = 64 bf16 = one 128-byte row, so the plane has the size and the 128-byte swizzle of the fp32 tile it sits
// behind; only K-major tiles are handled.  `raw` holds the A tile (A_BYTES) followed by the B tile.
template <int A_BYTES, int RAW_BYTES, int NTHREADS>
__device__ __forceinline__ void split_stage_bf16(uint8_t* raw, int tid) {
  static_assert(NTHREADS == 128 && A_BYTES % 2048 == 0 && (RAW_BYTES - A_BYTES) % 2048 == 0, "16 rows per sweep");
  // Thread t handles the 16-byte chunk t & 7 of row (t >> 3) + 16 j: row & 7 and the chunk, hence the K slice and
  // every swizzled offset, are the same in all its iterations; only the row advances (2048 bytes per sweep).
  const int r7 = (tid >> 3) & 7;
  const int cl = (tid & 7) ^ r7;               // logical chunk = 4 consecutive k
  const int g = cl >> 1, half = cl & 1;        // 8-wide K slice, and which half of it
  const int row_off = (tid >> 3) * 128;
  const int c_even = ((2 * g) ^ r7) << 4, c_odd = ((2 * g + 1) ^ r7) << 4;
  auto sweep = [&](const uint8_t* src, uint8_t* dst_lo, uint8_t* dst_hi) {
    const float4 x = *reinterpret_cast<const float4*>(src);
    const float h0 = __uint_as_float(__float_as_uint(x.x) & 0xffffe000u), h1 = __uint_as_float(__float_as_uint(x.y) & 0xffffe000u);
    const float h2 = __uint_as_float(__float_as_uint(x.z) & 0xffffe000u), h3 = __uint_as_float(__float_as_uint(x.w) & 0xffffe000u);
    uint2 lo, hi;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo.x) : "f"(x.y - h1), "f"(x.x - h0));   // upper half <- first operand
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo.y) : "f"(x.w - h3), "f"(x.z - h2));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi.x) : "f"(h1), "f"(h0));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi.y) : "f"(h3), "f"(h2));
    *reinterpret_cast<uint2*>(dst_lo) = lo;
    *reinterpret_cast<uint2*>(dst_hi) = hi;
  };
  const uint8_t* src = raw + tid * 16;
  uint8_t* plane = raw + RAW_BYTES + row_off + half * 8;
#pragma unroll
  for (int j = 0; j < A_BYTES / 2048; ++j)                      // A: [lo | hi]
    sweep(src + j * 2048, plane + j * 2048 + c_even, plane + j * 2048 + c_odd);
#pragma unroll
  for (int j = A_BYTES / 2048; j < RAW_BYTES / 2048; ++j)       // B: [hi | lo]
    sweep(src + j * 2048, plane + j * 2048 + c_odd, plane + j * 2048 + c_even);
}

// Store phase of the epilogue.  Each lane holds one output row (NC columns of it) in `acc`.  A
// 32 x 32 block goes through a per-warp shared-memory tile (16-byte chunks XOR-swizzled by row) so
// that every global access of C, Z and bias is a run of whole 128-byte lines instead of 32 scattered
// 16-byte pieces.  `row_base` is the first of the warp's 32 rows, `n0` its first column; element
// (row, col) of matrix b goes to t.C[tile_off + row * t.ldc + col], or where p.omap places it.
template <int NC>
__device__ __forceinline__ void epilogue_store_rows(const UmmaParams& p, const StoreTarget& t, const float (&acc)[NC],
                                              float* stage, int b, long long tile_off, int row_base, int n0, int lane) {
  const bool heavy = t.act != ACT_IDENTITY && t.act != ACT_RELU;
#pragma unroll
  for (int g = 0; g < NC / 32; ++g) {
    const int col0 = n0 + g * 32;
    if (col0 >= p.N) break;  // warp-uniform
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
      const float4 v4 = make_float4(acc[g * 32 + 4 * j4], acc[g * 32 + 4 * j4 + 1], acc[g * 32 + 4 * j4 + 2],
                                    acc[g * 32 + 4 * j4 + 3]);
      *reinterpret_cast<float4*>(stage + lane * 32 + ((j4 ^ (lane & 7)) << 2)) = v4;
    }
    __syncwarp();
    if (t.vec_ok && col0 + 32 <= p.N) {
      if (t.mapped)   epilogue_store_block_vec<true, true>(p, t, stage, b, tile_off, row_base, col0, lane);
      else if (heavy) epilogue_store_block_vec<true, false>(p, t, stage, b, tile_off, row_base, col0, lane);
      else            epilogue_store_block_vec<false, false>(p, t, stage, b, tile_off, row_base, col0, lane);
    } else {
      // ragged right edge or rows that are not 16-byte aligned: one column per lane
      const int col = col0 + lane;
      if (col < p.N) {
        const float bv = t.bias ? __ldg(t.bias + col) : 0.0f;
        for (int r = 0; r < 32; ++r) {
          const int row = row_base + r;
          if (row >= p.M) break;
          const float a1 = stage[r * 32 + ((((lane >> 2) ^ (r & 7)) << 2) | (lane & 3))];
          long long off = tile_off + static_cast<long long>(row) * t.ldc + col;
          if (t.mapped) off = out_offset(p.omap, b, row, col);
          float o = t.alpha * a1;
          if (t.beta != 0.0f) o = fmaf(t.beta, t.C[off], o);
          o += bv;
          if (t.Z) t.Z[off] = o;
          t.C[off] = act_forward(t.act, o, t.act_alpha);
        }
      }
    }
    __syncwarp();
  }
}

// Coalesced read of a 32 x 32 block of a row-major matrix (rows 16-byte aligned) through the warp's shared-memory
// tile, the mirror image of the store phase: afterwards lane l holds row l of the block in `out`.  Rows at or
// beyond `rows_valid` and columns at or beyond `cols_valid` read as 0.
__device__ __forceinline__ void epilogue_load_block(const float* src, int ld, int rows_valid, int cols_valid, float* stage,
                                                    int lane, float (&out)[32]) {
  const int c4 = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + (lane >> 3);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows_valid && 4 * c4 < cols_valid) v = *reinterpret_cast<const float4*>(src + static_cast<long long>(r) * ld + 4 * c4);
    *reinterpret_cast<float4*>(stage + r * 32 + ((c4 ^ (r & 7)) << 2)) = v;
  }
  __syncwarp();
#pragma unroll
  for (int j4 = 0; j4 < 8; ++j4) {
    const float4 v = *reinterpret_cast<const float4*>(stage + lane * 32 + ((j4 ^ (lane & 7)) << 2));
    out[4 * j4] = v.x; out[4 * j4 + 1] = v.y; out[4 * j4 + 2] = v.z; out[4 * j4 + 3] = v.w;
  }
  __syncwarp();
}

// beta * C folded into the accumulator at the start of a tile: the epilogue warps, idle until the first partial sum
// is ready, read their rows of C (coalesced, through the shared-memory tile) while the tensor core works, and start
// the register accumulator at (beta / alpha) * C instead of 0.  The store phase then has nothing to read: with one
// tile per SM nothing would hide those reads there (measured: 2048 x 1536 x 768 with beta = 1 took 55 us against 37 us
// with beta = 0).  The extra rounding is one ulp of beta * C.  Returns false when the fold does not apply (the store
// phase then reads C as before): alpha = 0, rows not 16-byte aligned, a mapped result, partial sums, a row operation.
template <int NC>
__device__ __forceinline__ bool epilogue_fold_c(const UmmaParams& p, float (&acc)[NC], float* stage, int b, int split,
                                                int row_base, int n0, int lane) {
  if (p.beta == 0.0f || p.alpha == 0.0f || !p.vec_ok || p.omap.on || p.row_op != ROW_NONE ||
      (split >= 0 && p.partial != nullptr))
    return false;
  const float f = p.beta / p.alpha;
  const float* cb = p.C + static_cast<long long>(b) * p.strideC + static_cast<long long>(row_base) * p.ldc + n0;
  const int rows_valid = p.M - row_base;
#pragma unroll
  for (int g = 0; g < NC / 32; ++g) {
    const int cols_valid = p.N - (n0 + g * 32);
    if (cols_valid <= 0) break;   // warp-uniform
    float y[32];
    epilogue_load_block(cb + g * 32, p.ldc, rows_valid, cols_valid, stage, lane, y);
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[g * 32 + j] = f * y[j];
  }
  return true;
}

// Row operation of the attention products.  The launcher guarantees one tile column, so an output row lies in this
// tile: in one lane's NC registers (GROUPS = 1), or split between the two warps that read the same TMEM lanes
// (GROUPS = 2: warp 4 + q holds columns [0, NC), warp 8 + q columns [NC, 2 NC)); those two exchange the row maximum
// and the row sum through shared memory (`xch`, [2][128] floats: one slot per group and row) and meet at the named
// barrier 1 + q, once before a slot is overwritten and once before it is read.  Two warps per row halve the serial work of a lane and give every scheduler a second warp to
// hide latencies with.  Rows are 16-byte aligned and N is a multiple of 4.  On return acc holds the values to store.
//   ROW_SOFTMAX       acc = softmax(mask(alpha * acc + bias)) over the N valid columns: the causal overwrite with -1e12
//                     (Prod/CPU/CpuTensor.cs:3037-3052) and CpuTensorActivationFunctions.Softmax (:19-46).
//                     The exponential is the hardware's ex2 (relative error 2^-22) and the division a multiplication
//                     by the reciprocal of the row sum; maximum and sum run as four independent chains.
//   ROW_SOFTMAX_GRAD  acc = y * (g - sum_j g_j * y_j) with g = alpha * acc, y = aux row: the softmax Jacobian
//                     cudnnSoftmaxBackward applies (Prod/GPU/GpuTensor.cs:445-490)
__device__ __forceinline__ void row_pair_barrier(int q) { asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory"); }

// Both warps of a row pair must take the same decision before a row operation, or one would wait at the named
// barrier for a partner that has left: each contributes its own `ok` (every wait behind it is bounded, so both
// always arrive here) and both continue only if both are.  Slot use: [group][q * 32 + lane], like the exchanges.
__device__ __forceinline__ bool row_pair_all(float* xch, int q, int group, int lane, bool ok) {
  row_pair_barrier(q);
  xch[group * 128 + q * 32 + lane] = ok ? 1.0f : 0.0f;
  row_pair_barrier(q);
  return ok && xch[(group ^ 1) * 128 + q * 32 + lane] != 0.0f;
}

// This lane's value against the value of the lane that holds the other half of the row.
__device__ __forceinline__ float row_pair_exchange(float* xch, int q, int group, int lane, float mine) {
  row_pair_barrier(q);                       // the partner has read what the slot held before
  xch[group * 128 + q * 32 + lane] = mine;
  row_pair_barrier(q);
  return xch[(group ^ 1) * 128 + q * 32 + lane];
}

template <int NC, int GROUPS>
__device__ __forceinline__ void epilogue_row_op(const UmmaParams& p, float (&acc)[NC], float* stage, float* xch, int b,
                                                int row_base, int col_base, int q, int group, int lane) {
  const int ncols = max(0, min(NC, p.N - col_base));   // valid columns among this lane's NC
  const int row = row_base + lane;
  if (p.row_op == ROW_SOFTMAX) {
    const int limit = p.causal ? row : 0x7fffffff;   // columns > limit are masked
    float m4[4] = {-3.402823466e38f, -3.402823466e38f, -3.402823466e38f, -3.402823466e38f};
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float v = p.alpha * acc[j];
      if (p.bias != nullptr && j < ncols) v += __ldg(p.bias + col_base + j);   // Dense + Softmax
      v = (col_base + j > limit) ? -1e12f : v;
      v = (j < ncols) ? v : -3.402823466e38f;
      acc[j] = v;
      m4[j & 3] = fmaxf(m4[j & 3], v);
    }
    float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
    if (GROUPS == 2) mx = fmaxf(mx, row_pair_exchange(xch, q, group, lane, mx));
    const float c = mx * 1.4426950408889634f;
    float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float e;
      asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(acc[j], 1.4426950408889634f, -c)));
      e = (j < ncols) ? e : 0.0f;
      acc[j] = e;
      s4[j & 3] += e;
    }
    float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
    if (GROUPS == 2) {
      const float other = row_pair_exchange(xch, q, group, lane, sum);
      sum = group == 0 ? sum + other : other + sum;   // same order in both warps: identical results
    }
    const float inv = 1.0f / sum;
#pragma unroll
    for (int j = 0; j < NC; ++j) acc[j] *= inv;
  } else {
    const float* yb = p.aux + static_cast<long long>(b) * p.strideC + static_cast<long long>(row_base) * p.ldc + col_base;
    const int rows_valid = p.M - row_base;
    float d4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int g = 0; g < NC / 32; ++g) {
      if (g * 32 >= ncols) break;   // warp-uniform
      float y[32];
      epilogue_load_block(yb + g * 32, p.ldc, rows_valid, ncols - g * 32, stage, lane, y);
#pragma unroll
      for (int j = 0; j < 32; ++j) d4[j & 3] = fmaf(p.alpha * acc[g * 32 + j], y[j], d4[j & 3]);
    }
    float dot = (d4[0] + d4[1]) + (d4[2] + d4[3]);
    if (GROUPS == 2) {
      const float other = row_pair_exchange(xch, q, group, lane, dot);
      dot = group == 0 ? dot + other : other + dot;
    }
#pragma unroll
    for (int g = 0; g < NC / 32; ++g) {
      if (g * 32 >= ncols) break;
      float y[32];
      epilogue_load_block(yb + g * 32, p.ldc, rows_valid, ncols - g * 32, stage, lane, y);   // second read: L1 / L2
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[g * 32 + j] = y[j] * (p.alpha * acc[g * 32 + j] - dot);
    }
  }
}

// Final store of one work unit: the fused epilogue into C, or (split >= 0) the raw partial sums into
// the workspace.  `tile_row0`/`tile_col0` are the first row and column of the unit's whole tile,
// `tile_elems` the size of that tile in the tiled workspace layout (rows x BN), `bn` its row pitch there.
// `alpha` / `bias` are p.alpha / p.bias, or 1 / nullptr when a row operation has already applied them; `beta` is
// p.beta, or 0 when beta * C is already part of the accumulator.
template <int NC>
__device__ __forceinline__ void epilogue_store_unit(const UmmaParams& p, float alpha, float beta, const float* bias,
                                                    const float (&acc)[NC], float* stage,
                                                    int b, int n_tiles, int tile, int split, int tile_row0, int tile_col0,
                                                    int bn, int row_base, int n0, int lane, long long c_shift = 0) {
  // one call of the store phase (its code is long: a second copy costs instruction-cache misses); the
  // partial-sum case redirects it to the workspace
  StoreTarget t = {p.C + c_shift, p.Z, bias, alpha, beta, p.act, p.ldc, p.vec_ok, p.omap.on, p.act_alpha};
  long long off = static_cast<long long>(b) * p.strideC;
  if (split >= 0 && p.partial != nullptr) {
    t.C = p.partial;
    t.mapped = 0;     // partial sums have their own layout; the reduction pass applies the placement
    t.alpha = 1.0f; t.beta = 0.0f; t.bias = nullptr; t.Z = nullptr; t.act = ACT_IDENTITY;
    if (p.partial_tiled) {
      const int tail = n_tiles - p.whole_tiles;
      const long long slot = static_cast<long long>(split) * tail + (tile - p.whole_tiles);
      t.ldc = bn;
      t.vec_ok = 1;
      off = slot * p.partial_stride - (static_cast<long long>(tile_row0) * bn + tile_col0);
    } else {
      t.ldc = p.N;
      t.vec_ok = (p.N % 4 == 0) ? 1 : 0;
      off = static_cast<long long>(split) * p.partial_stride + static_cast<long long>(b) * p.M * p.N;
    }
  }
  epilogue_store_rows<NC>(p, t, acc, stage, b, off, row_base, n0, lane);
}

// Store phase of a kernel that ran the transposed problem (p.store_t): the lane's row of the tile is a column of
// the caller's matrix, so for every tile column the 32 lanes of a warp write 32 consecutive floats of one row of C.
// The bias runs along the tile's rows.
template <int NC>
__device__ __forceinline__ void epilogue_store_transposed(const UmmaParams& p, float beta, const float (&acc)[NC], int b,
                                                          int row_base, int n0, int lane) {
  const int r = row_base + lane;
  if (r >= p.M) return;
  const float bv = p.bias ? __ldg(p.bias + r) : 0.0f;
  const long long base = static_cast<long long>(b) * p.strideC + r;
#pragma unroll       // fully: acc must stay in registers
  for (int j = 0; j < NC; ++j) {
    const int c = n0 + j;
    if (c >= p.N) break;
    const long long off = base + static_cast<long long>(c) * p.ldc;
    float o = p.alpha * acc[j];
    if (beta != 0.0f) o = fmaf(beta, p.C[off], o);
    o += bv;
    if (p.Z) p.Z[off] = o;
    p.C[off] = act_forward_compact(p.act, o, p.act_alpha);
  }
}

// beta * C of a transposed store, read while the products run (see epilogue_fold_c): acc starts at (beta / alpha) * C.
template <int NC>
__device__ __forceinline__ bool epilogue_fold_c_transposed(const UmmaParams& p, float (&acc)[NC], int b, int row_base,
                                                           int n0, int lane) {
  if (p.beta == 0.0f || p.alpha == 0.0f) return false;
  const int r = row_base + lane;
  const float f = p.beta / p.alpha;
  const float* cb = p.C + static_cast<long long>(b) * p.strideC + r;
  // all loads first, then their uses: issued one after the other they would cost a memory latency each, and the
  // tensor core waits for the accumulator buffers this warp has not drained yet
  const int rc = r < p.M ? r : 0;     // rows past the edge read a valid address; their values are never stored
  float c[NC];
#pragma unroll
  for (int j = 0; j < NC; ++j) {
    const int col = n0 + j < p.N ? n0 + j : p.N - 1;
    c[j] = *(cb - r + rc + static_cast<long long>(col) * p.ldc);
  }
#pragma unroll
  for (int j = 0; j < NC; ++j) acc[j] = f * c[j];
  return true;
}

// 3xTF32 operand split of one landed stage: lo = tf32(x - hi) goes to the second plane, RAW_BYTES
// after the raw tile, at the same (swizzled) offset.
template <int RAW_BYTES, int NTHREADS>
__device__ __forceinline__ void split_stage(uint8_t* raw, int tid, int rewrite_hi) {
#pragma unroll 8
  for (int i = tid; i < RAW_BYTES / 16; i += NTHREADS) {
    float4 x = *reinterpret_cast<const float4*>(raw + i * 16);
    uint4 hi, lo;
    if (rewrite_hi) {
      hi.x = to_tf32_rna(x.x); hi.y = to_tf32_rna(x.y); hi.z = to_tf32_rna(x.z); hi.w = to_tf32_rna(x.w);
    } else {
      // The tensor core reads only the top 19 bits of each word: the raw tile is the hi plane.
      hi.x = __float_as_uint(x.x) & 0xffffe000u; hi.y = __float_as_uint(x.y) & 0xffffe000u;
      hi.z = __float_as_uint(x.z) & 0xffffe000u; hi.w = __float_as_uint(x.w) & 0xffffe000u;
    }
    lo.x = to_tf32_rna(x.x - __uint_as_float(hi.x));
    lo.y = to_tf32_rna(x.y - __uint_as_float(hi.y));
    lo.z = to_tf32_rna(x.z - __uint_as_float(hi.z));
    lo.w = to_tf32_rna(x.w - __uint_as_float(hi.w));
    if (rewrite_hi) *reinterpret_cast<uint4*>(raw + i * 16) = hi;
    *reinterpret_cast<uint4*>(raw + RAW_BYTES + i * 16) = lo;
  }
}

// Operand split of one landed stage when A goes to the tensor core from tensor memory.  Thread `tid` of the 128
// split threads owns row `tid` of the A tile: it reads the row's 32 K values from shared memory (K-major tile: eight
// swizzled 16-byte chunks; MN-major tile: one word per K row of the 32-wide chunk its row lies in, 32-byte atoms
// XOR-swizzled by K row & 3), and writes them -- raw, the tensor core truncates to TF32 itself -- to TMEM columns
// [0, 32) of the stage and lo = tf32(x - hi) to columns [32, 64), lane = row.  The B tile is split in shared memory
// as before, its lo plane right behind it.
template <class T>
__device__ __forceinline__ void split_stage_ts(uint8_t* stage, uint32_t tmem_a, int tid, int a_mn) {
  uint32_t x[32], lo[32];
  if (!a_mn) {
    const uint8_t* row = stage + tid * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(row + ((c ^ (tid & 7)) << 4));
      x[4 * c] = v.x; x[4 * c + 1] = v.y; x[4 * c + 2] = v.z; x[4 * c + 3] = v.w;
    }
  } else {
    const uint8_t* chunk = stage + (tid >> 5) * T::MNMAJ_CHUNK_BYTES + (tid & 7) * 4;
    const int atom = (tid >> 3) & 3;
#pragma unroll
    for (int k = 0; k < 32; ++k) x[k] = *reinterpret_cast<const uint32_t*>(chunk + k * 128 + ((atom ^ (k & 3)) << 5));
  }
#pragma unroll
  for (int j = 0; j < 32; ++j)
    lo[j] = to_tf32_rna(__uint_as_float(x[j]) - __uint_as_float(x[j] & 0xffffe000u));
  const uint32_t lane_base = static_cast<uint32_t>(tid & ~31) << 16;     // this warp's TMEM lane quarter
  tmem_st_32x32(tmem_a + lane_base, x);
  tmem_st_32x32(tmem_a + lane_base + 32, lo);
  uint8_t* b_raw = stage + T::A_BYTES;
#pragma unroll 4
  for (int i = tid; i < T::B_BYTES / 16; i += 128) {
    const float4 v = *reinterpret_cast<const float4*>(b_raw + i * 16);
    uint4 l;
    l.x = to_tf32_rna(v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u));
    l.y = to_tf32_rna(v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u));
    l.z = to_tf32_rna(v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u));
    l.w = to_tf32_rna(v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u));
    *reinterpret_cast<uint4*>(b_raw + T::B_BYTES + i * 16) = l;
  }
  tmem_st_wait();
}

// One operand tile built in shared memory by the loader warps, in the layout TMA delivers, with asynchronous 4-byte
// copies (cp.async): no alignment beyond a float's is needed, nothing is staged in registers, and a thread keeps
// the copies of several stages in flight (the loader loop waits for a stage's copies only when it signals it).
//   K-major (`mn` = 0): `rows` tile rows (M or N index) of 32 K values; row r sits at r * 128 bytes, its 16-byte chunk
//       c at position c ^ (r & 7).  Source element (r, k) = src[(r0 + r) * ld + k0 + k].
//   MN-major (`mn` = 1): 32 K rows of `rows` contiguous M/N values, in chunks of 32 values: chunk j at j * 4096 bytes,
//       K row k at k * 128, 32-byte atom a at position a ^ (k & 3).  Source element (k, r) = src[(k0 + k) * ld + r0 + r].
// A warp copies 32 consecutive source floats per instruction (one 128-byte line).  Elements outside the matrix are
// zero-filled (source size 0 with the address clamped into the matrix), as TMA's out-of-bounds fill does.
__device__ __forceinline__ void cp_async_4(uint32_t smem_dst, const float* src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void sw_issue_tile(uint8_t* dst, const float* src, long long ld, int mn, int rows, int r0,
                                              int r_limit, int k0, int k_limit, int tid, int nthreads) {
  const uint32_t d0 = smem_u32(dst);
  const int lane = tid & 31, w = tid >> 5, nw = nthreads >> 5;
  if (!mn) {
    // one warp instruction = one tile row: lane = K index
    const bool k_ok = k0 + lane < k_limit;
    const uint32_t in_row = ((lane >> 2) << 4) | ((lane & 3) << 2);          // chunk lane / 4, word lane % 4
    const float* ptr = src + static_cast<long long>(r0 + w) * ld + k0 + lane;
    const long long step = static_cast<long long>(nw) * ld;
#pragma unroll 4
    for (int r = w; r < rows; r += nw, ptr += step) {
      const bool ok = k_ok && r0 + r < r_limit;
      cp_async_4(d0 + r * 128 + (in_row ^ ((r & 7) << 4)), ok ? ptr : src, ok ? 4u : 0u);
    }
  } else {
    // one warp instruction = 32 consecutive M/N values of one K row: lane = position in the 32-wide chunk.
    // Warp w takes K rows w, w + nw, ... of every chunk.
    const int chunks = rows >> 5;
    const uint32_t in_row = ((lane >> 3) << 5) | ((lane & 7) << 2);          // atom lane / 8, word lane % 8
    const long long step = static_cast<long long>(nw) * ld;
    for (int j = 0; j < chunks; ++j) {
      const int col = r0 + 32 * j + lane;
      const bool col_ok = col < r_limit;
      const float* ptr = src + static_cast<long long>(k0 + w) * ld + col;
#pragma unroll 4
      for (int kr = w; kr < 32; kr += nw, ptr += step) {
        const bool ok = col_ok && k0 + kr < k_limit;
        cp_async_4(d0 + j * 4096 + kr * 128 + (in_row ^ ((kr & 3) << 5)), ok ? ptr : src, ok ? 4u : 0u);
      }
    }
  }
}

// The tensor core adds into its fp32 accumulator with truncation, so a long K loop drifts towards
// zero by about 1e-8 * K (relative to sqrt(K)).  The MMA warp therefore accumulates only
// `chunk_kblocks` k-blocks in TMEM; the epilogue warps add every such partial sum into fp32
// registers (round-to-nearest), alternating between the two TMEM buffers so that the tensor core
// never waits for them.
// ROWOP instantiates the epilogue with the row operations of attention (epilogue_row_op); the plain
// instantiation carries none of their code or registers.
template <class T, bool ROWOP, int CLUSTER, bool GROUPED>
__device__ __forceinline__ void umma_gemm_core(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2,
                                               const CUtensorMap& tmB2, const UmmaParams& p) {
  static_assert(!GROUPED || (!ROWOP && CLUSTER == 1 && !T::SWLOAD && !T::TS), "the grouped form is the plain product");
  constexpr int BM = T::BM, BN = T::BN, BK = T::BK, STAGES = T::STAGES;
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[STAGES];    // TMA bytes landed
  __shared__ uint64_t split_bar[STAGES];   // hi/lo planes written (3xTF32)
  __shared__ uint64_t empty_bar[STAGES];   // MMAs that read the stage retired
  __shared__ uint64_t acc_full_bar[2];     // partial sum complete in TMEM
  __shared__ uint64_t acc_empty_bar[2];    // partial sum moved to registers
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;
  __shared__ float row_xch[ROWOP ? 2 * 128 : 1];   // row maximum / sum exchange of the row operations
  __shared__ uint64_t xchg_bar;            // CLUSTER: the other CTAs' partial sums of the rows this CTA stores are published
  static_assert(CLUSTER == 1 || CLUSTER == 2 || CLUSTER == 4, "clusters of 2 or 4 CTAs");
  static_assert(CLUSTER == 1 || (!ROWOP && !T::TS && !T::SWLOAD), "the cluster form is the plain product");
  static_assert(4 * T::EPI_GROUPS * 32 * T::EPI_COLS * 4 <= T::RING_BYTES, "partial sums are published in the operand ring");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* ring = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
  if (threadIdx.x == 0) SNB_STAMP(p, 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], T::SWLOAD ? T::N_LOAD_THREADS / 32 : 1);     // TMA bytes, or one arrival per loader warp
      mbar_init(&split_bar[s], T::SPLIT ? T::N_SPLIT_THREADS / 32 : 1);   // one arrival per split warp
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full_bar[b], 1);
      mbar_init(&acc_empty_bar[b], T::EPI_THREADS / 32);   // one arrival per epilogue warp
    }
    // every other CTA's warps of the row quarters this CTA owns arrive once
    mbar_init(&xchg_bar, CLUSTER > 1 ? (CLUSTER - 1) * (4 / CLUSTER) * T::EPI_GROUPS : 1);
    abort_flag = 0;
    fence_mbar_init();
    if (!T::SWLOAD) {
      prefetch_tmap(&tmA);
      prefetch_tmap(&tmB);
      if (GROUPED) {
        prefetch_tmap(&tmA2);
        prefetch_tmap(&tmB2);
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_holder, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  if (CLUSTER > 1) cluster_sync_all();   // the barriers of every CTA of the cluster exist before anyone signals them
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_holder;
  volatile int* abortp = &abort_flag;
  // Everything above touched only this CTA's shared memory, TMEM and kernel parameters, so it may overlap the
  // tail of the previous kernel in the stream; everything below reads or writes global memory.
  if (threadIdx.x == 0) SNB_STAMP(p, 1);
  allow_dependent_launch();
  grid_dependency_wait();
  if (threadIdx.x == 0) SNB_STAMP(p, 2);

  const int n_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int total_tiles = p.whole_tiles + (n_tiles - p.whole_tiles) * p.splits;   // work units

  if (warp < 4) {
    reg_dealloc<T::REGS_CTRL>();
    if (warp == 0 && lane == 0 && !T::SWLOAD) {
      // ---------------------------------------------------------------- TMA producer
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int tile, split, kb_begin, kb_end, b, tm, tn;
        unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
        tile_coords(tile, p.tiles_m, p.tiles_n, b, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        const bool second = GROUPED && b >= p.group_batch;
        const CUtensorMap* mapA = second ? &tmA2 : &tmA;
        const CUtensorMap* mapB = second ? &tmB2 : &tmB;
        if (second) b -= p.group_batch;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) { ok = false; break; }
          uint8_t* a_dst = ring + s * T::STAGE_BYTES;
          uint8_t* b_dst = a_dst + T::A_BYTES;
          mbar_arrive_expect_tx(&full_bar[s], T::RAW_BYTES);
          const int k0 = kb * BK;
          if (t == blockIdx.x && kb == kb_begin) SNB_STAMP(p, 3);
          if (!p.a_mn) {
            tma_load_3d(a_dst, mapA, &full_bar[s], k0, m0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 32; ++j)
              tma_load_3d(a_dst + j * T::MNMAJ_CHUNK_BYTES, mapA, &full_bar[s], m0 + 32 * j, k0, b);
          }
          if (!p.b_mn) {
            tma_load_3d(b_dst, mapB, &full_bar[s], k0, n0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 32; ++j)
              tma_load_3d(b_dst + j * T::MNMAJ_CHUNK_BYTES, mapB, &full_bar[s], n0 + 32 * j, k0, b);
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      const uint32_t idesc = make_idesc_tf32(BM, BN, T::TS ? 0 : p.a_mn, p.b_mn);   // A in TMEM is always K-major
      const uint32_t a_step = p.a_mn ? 1024u : 32u;   // bytes per K = 8 slice
      const uint32_t b_step = p.b_mn ? 1024u : 32u;
      const uint32_t a_lbo = p.a_mn ? T::MNMAJ_CHUNK_BYTES : 16u;
      const uint32_t b_lbo = p.b_mn ? T::MNMAJ_CHUNK_BYTES : 16u;
      const uint32_t a_sbo = p.a_mn ? T::MNMAJ_SBO : T::KMAJ_SBO;
      const uint32_t b_sbo = p.b_mn ? T::MNMAJ_SBO : T::KMAJ_SBO;
      const uint32_t a_lay = p.a_mn ? T::MNMAJ_LAYOUT : T::KMAJ_LAYOUT;
      const uint32_t b_lay = p.b_mn ? T::MNMAJ_LAYOUT : T::KMAJ_LAYOUT;
      const uint64_t desc_a0 = make_smem_desc(0, a_lbo, a_sbo, a_lay), desc_b0 = make_smem_desc(0, b_lbo, b_sbo, b_lay);
      const uint32_t a_step16 = a_step >> 4, b_step16 = b_step >> 4;
      int s = 0;
      uint32_t ph = 0;
      uint32_t acc_ph = 0;  // bit b = phase of TMEM buffer b
      uint32_t chunk_id = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int tile, split, kb_begin, kb_end;
        unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
        for (int kb0 = kb_begin; kb0 < kb_end && ok; kb0 += p.chunk_kblocks, ++chunk_id) {
          const int buf = chunk_id & 1;
          if (!mbar_wait(&acc_empty_bar[buf], ((acc_ph >> buf) & 1u) ^ 1u, abortp)) { ok = false; break; }
          acc_ph ^= 1u << buf;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * BN;
          const int kb1 = min(kb_end, kb0 + p.chunk_kblocks);
          for (int kb = kb0; kb < kb1; ++kb) {
            uint64_t* ready = T::SPLIT ? &split_bar[s] : &full_bar[s];
            if (!mbar_wait(ready, ph, abortp)) { ok = false; break; }
            if (t == blockIdx.x && kb == kb_begin) SNB_STAMP(p, 5);
            if (t == blockIdx.x && kb - kb_begin < 8) SNB_STAMP(p, 16 + 2 * (kb - kb_begin));
            tc_fence_after_sync();
            const uint32_t a_hi = smem_u32(ring + s * T::STAGE_BYTES);
            const uint32_t b_hi = a_hi + T::A_BYTES;
            const uint32_t a_tmem = tmem_base + T::TS_A_COL0 + s * T::TS_A_COLS;   // TS: hi plane, lo plane 32 columns on
            if (!T::TS && !kSlowIssue) {
              // Descriptors differ from slice to slice and from plane to plane only in their start-address field (bits
              // 0-13, in 16-byte units), so they are formed by additions to one descriptor per operand and K block:
              // the issuing lane spends a few instructions per tcgen05.mma instead of rebuilding every descriptor.
              // (the address field holds bits 4-17 of the CTA-relative address: in a cluster launch shared-memory
              // addresses carry the CTA's rank in higher bits, which must not spill into the next field)
              const uint64_t da0 = desc_a0 + ((a_hi & 0x3ffffu) >> 4), db0 = desc_b0 + ((b_hi & 0x3ffffu) >> 4);
#pragma unroll
              for (int ks = 0; ks < BK / kUmmaK; ++ks) {
                const uint64_t da_hi = da0 + ks * a_step16, db_hi = db0 + ks * b_step16;
                const uint32_t first = (kb == kb0 && ks == 0) ? 0u : 1u;
                if (T::SPLIT) {
                  umma_tf32_ss(d_tmem, da_hi + (T::RAW_BYTES >> 4), db_hi, idesc, first);
                  umma_tf32_ss(d_tmem, da_hi, db_hi + (T::RAW_BYTES >> 4), idesc, 1u);
                  umma_tf32_ss(d_tmem, da_hi, db_hi, idesc, 1u);
                } else {
                  umma_tf32_ss(d_tmem, da_hi, db_hi, idesc, first);
                }
              }
            } else
#pragma unroll
            for (int ks = 0; ks < BK / kUmmaK; ++ks) {
              const uint64_t da_hi = make_smem_desc(a_hi + ks * a_step, a_lbo, a_sbo, a_lay);
              const uint64_t db_hi = make_smem_desc(b_hi + ks * b_step, b_lbo, b_sbo, b_lay);
              const uint32_t first = (kb == kb0 && ks == 0) ? 0u : 1u;
              if (T::TS) {
                const uint64_t db_lo = make_smem_desc(b_hi + T::B_LO_OFFSET + ks * b_step, b_lbo, b_sbo, b_lay);
                umma_tf32_ts(d_tmem, a_tmem + BK + ks * kUmmaK, db_hi, idesc, first);
                umma_tf32_ts(d_tmem, a_tmem + ks * kUmmaK, db_lo, idesc, 1u);
                umma_tf32_ts(d_tmem, a_tmem + ks * kUmmaK, db_hi, idesc, 1u);
              } else if (T::SPLIT) {
                const uint64_t da_lo = make_smem_desc(a_hi + T::RAW_BYTES + ks * a_step, a_lbo, a_sbo, a_lay);
                const uint64_t db_lo = make_smem_desc(b_hi + T::RAW_BYTES + ks * b_step, b_lbo, b_sbo, b_lay);
                umma_tf32_ss(d_tmem, da_lo, db_hi, idesc, first);
                umma_tf32_ss(d_tmem, da_hi, db_lo, idesc, 1u);
                umma_tf32_ss(d_tmem, da_hi, db_hi, idesc, 1u);
              } else {
                umma_tf32_ss(d_tmem, da_hi, db_hi, idesc, first);
              }
            }
            umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
            if (t == blockIdx.x && kb - kb_begin < 8) SNB_STAMP(p, 17 + 2 * (kb - kb_begin));
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
          if (ok) umma_commit(&acc_full_bar[buf]);
        }
        if (t == blockIdx.x) SNB_STAMP(p, 6);
      }
    }
    __syncwarp();
  } else if (warp < 4 + 4 * T::EPI_GROUPS) {
    // ------------------------------------------------------------------ epilogue
    reg_alloc<T::REGS_EPI>();
    constexpr int NC = T::EPI_COLS;          // columns this warp owns
    const int q = warp & 3;                  // TMEM lane quarter this warp may read
    const int col_base = ((warp - 4) >> 2) * NC;
    uint32_t acc_ph = 0;
    uint32_t chunk_id = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int tile, split, kb_begin, kb_end, b, tm, tn;
      unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
      tile_coords(tile, p.tiles_m, p.tiles_n, b, tm, tn);
      const int n_chunks = (kb_end - kb_begin + p.chunk_kblocks - 1) / p.chunk_kblocks;
      float* stage = reinterpret_cast<float*>(ring + T::RING_BYTES) + (warp - 4) * (T::EPI_STAGE_BYTES / 4);
      float acc[NC];
#pragma unroll
      for (int j = 0; j < NC; ++j) acc[j] = 0.0f;
      // CLUSTER: CTA r of the cluster stores the row quarters q with q * CLUSTER / 4 == r, summed over all K parts
      const int owner = CLUSTER > 1 ? q * CLUSTER / 4 : 0;
      const bool mine = CLUSTER == 1 || owner == static_cast<int>(cluster_ctarank());
      const bool c_folded =
          !mine ? false
          : (CLUSTER > 1 && p.store_t)
              ? epilogue_fold_c_transposed<NC>(p, acc, b, tm * BM + q * 32, tn * BN + col_base, lane)
              : epilogue_fold_c<NC>(p, acc, stage, b, split, tm * BM + q * 32, tn * BN + col_base, lane);
      for (int c = 0; c < n_chunks && ok; ++c, ++chunk_id) {
        const int buf = chunk_id & 1;
        if (!mbar_wait_warp(&acc_full_bar[buf], (acc_ph >> buf) & 1u, abortp)) { ok = false; break; }
        if (warp == 4 && lane == 0 && t == blockIdx.x && c == 0) SNB_STAMP(p, 7);
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
        if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
        if (warp == 4 && lane == 0 && t == blockIdx.x && c == n_chunks - 1) SNB_STAMP(p, 8);
      }
      if (ROWOP && T::EPI_GROUPS == 2) ok = row_pair_all(row_xch, q, (warp - 4) >> 2, lane, ok);
      if (!ok) break;
      if constexpr (CLUSTER > 1) {
        // The operand ring is free (the last products have retired and this CTA loads nothing more): each warp
        // owns 32 x NC floats of it, laid out [column quad][lane] so that neither side has bank conflicts.
        float4* slab = reinterpret_cast<float4*>(ring) + (warp - 4) * (NC / 4) * 32;
        if (!mine) {
#pragma unroll
          for (int j4 = 0; j4 < NC / 4; ++j4)
            slab[j4 * 32 + lane] = make_float4(acc[4 * j4], acc[4 * j4 + 1], acc[4 * j4 + 2], acc[4 * j4 + 3]);
          __syncwarp();
          if (lane == 0) mbar_arrive_release_cluster(map_to_cta(smem_u32(&xchg_bar), owner));
          continue;   // the owner stores these rows
        }
        if (!mbar_wait_acquire_cluster_warp(&xchg_bar, 0, abortp)) { ok = false; break; }
        const uint32_t rank = cluster_ctarank();
#pragma unroll
        for (uint32_t r = 0; r < CLUSTER; ++r) {       // fixed order: the sum does not depend on timing
          if (r == rank) continue;
          const uint32_t peer = map_to_cta(smem_u32(slab), r) + lane * 16;
#pragma unroll
          for (int j4 = 0; j4 < NC / 4; ++j4) {
            const float4 v = ld_shared_cluster_v4(peer + j4 * 512);
            acc[4 * j4] += v.x; acc[4 * j4 + 1] += v.y; acc[4 * j4 + 2] += v.z; acc[4 * j4 + 3] += v.w;
          }
        }
        if (p.store_t) {
          epilogue_store_transposed<NC>(p, c_folded ? 0.0f : p.beta, acc, b, tm * BM + q * 32, tn * BN + col_base, lane);
          continue;
        }
      }
      float alpha = p.alpha;
      const float* bias = p.bias;
      if (ROWOP) {   // this instantiation is launched for row operations only
        epilogue_row_op<NC, T::EPI_GROUPS>(p, acc, stage, row_xch, b, tm * BM + q * 32, col_base, q, (warp - 4) >> 2,
                                           lane);
        alpha = 1.0f;                      // the row operation has consumed both
        bias = nullptr;
      }
      epilogue_store_unit<NC>(p, alpha, c_folded ? 0.0f : p.beta, bias, acc, stage, b, n_tiles, tile, split, tm * BM, tn * BN,
                              BN, tm * BM + q * 32, tn * BN + col_base, lane,
                              (GROUPED && b >= p.group_batch) ? p.c_shift : 0);
      if (warp == 4 && lane == 0) SNB_STAMP(p, t == blockIdx.x ? 9 : 10);
    }
  } else if (T::SPLIT && threadIdx.x < T::LOAD_THREAD0) {
    // ------------------------------------------------------------------ hi / lo split
    reg_dealloc<T::REGS_SPLIT>();
    const int tid = threadIdx.x - T::SPLIT_THREAD0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int tile, split, kb_begin, kb_end;
      unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait_warp(&full_bar[s], ph, abortp)) { ok = false; break; }
        if (tid == 0 && t == blockIdx.x && kb == kb_begin) SNB_STAMP(p, 4);
        if (tid == 0 && t == blockIdx.x && kb - kb_begin < 8) SNB_STAMP(p, 32 + 2 * (kb - kb_begin));
        if constexpr (T::TS) {
          // the stage's TMEM columns are free: the producer refilled the stage only after the MMAs that read them retired
          split_stage_ts<T>(ring + s * T::STAGE_BYTES, tmem_base + T::TS_A_COL0 + s * T::TS_A_COLS, tid, p.a_mn);
          tc_fence_before_sync();
        } else {
          split_stage<T::RAW_BYTES, T::N_SPLIT_THREADS>(ring + s * T::STAGE_BYTES, tid, p.rewrite_hi);
        }
        fence_proxy_async_smem();   // make the generic-proxy stores visible to tcgen05.mma
        __syncwarp();
        if (lane == 0) mbar_arrive(&split_bar[s]);
        if (tid == 0 && t == blockIdx.x && kb - kb_begin < 8) SNB_STAMP(p, 33 + 2 * (kb - kb_begin));
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  }
  if (T::SWLOAD && threadIdx.x >= T::LOAD_THREAD0) {
    // ------------------------------------------------------------------ loader warps (operands TMA cannot load)
    reg_dealloc<T::REGS_LOAD>();
    const int tid = threadIdx.x - T::LOAD_THREAD0;
    constexpr int DEPTH = STAGES - 1 < 3 ? STAGES - 1 : 3;   // stages whose copies stay in flight behind the one being signalled
    int s = 0, s_signal = 0, pending = 0;
    uint32_t ph = 0;
    bool ok = true;
    // The copies of a stage are complete for this thread after cp.async.wait_group; the fence then orders them
    // before the tensor core's reads (async proxy), and one arrival per warp signals the stage.
    auto signal = [&]() {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_bar[s_signal]);
      if (++s_signal == STAGES) s_signal = 0;
      --pending;
    };
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int tile, split, kb_begin, kb_end, b, tm, tn;
      unit_decode(p, n_tiles, t, tile, split, kb_begin, kb_end);
      tile_coords(tile, p.tiles_m, p.tiles_n, b, tm, tn);
      const float* Ab = p.A + static_cast<long long>(b) * p.strideA;
      const float* Bb = p.B + static_cast<long long>(b) * p.strideB;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        // about to wait for the consumers: first hand over everything that is in flight, they may be waiting for it
        const bool must_wait = __shfl_sync(0xffffffffu, mbar_try_wait(&empty_bar[s], ph ^ 1) ? 0 : 1, 0) != 0;
        if (must_wait && pending > 0) {
          cp_async_wait<0>();
          while (pending > 0) signal();
        }
        if (!mbar_wait_warp(&empty_bar[s], ph ^ 1, abortp)) { ok = false; break; }
        uint8_t* a_dst = ring + s * T::STAGE_BYTES;
        sw_issue_tile(a_dst, Ab, p.lda, p.a_mn, BM, tm * BM, p.M, kb * BK, p.K, tid, T::N_LOAD_THREADS);
        sw_issue_tile(a_dst + T::A_BYTES, Bb, p.ldb, p.b_mn, BN, tn * BN, p.N, kb * BK, p.K, tid, T::N_LOAD_THREADS);
        cp_async_commit();
        ++pending;
        if (++s == STAGES) { s = 0; ph ^= 1; }
        if (pending > DEPTH) {
          cp_async_wait<DEPTH>();
          signal();
        }
      }
    }
    cp_async_wait<0>();           // the tail: everything has landed (also when the CTA is aborting)
    while (ok && pending > 0) signal();
  }

  // ---------------------------------------------------------------------- teardown
  if (threadIdx.x == 0) SNB_STAMP(p, 11);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
  // No CTA leaves while another may still read its shared memory.  Every thread of every CTA gets here: all waits
  // above are bounded.
  if (CLUSTER > 1) cluster_sync_all();
  if (threadIdx.x == 0 && abort_flag) atomicExch(p.error_word, 1);
  if (threadIdx.x == 0) SNB_STAMP(p, 12);
}

template <class T, bool ROWOP = false, int CLUSTER = 1>
__global__ void __launch_bounds__(T::THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const UmmaParams p) {
  umma_gemm_core<T, ROWOP, CLUSTER, false>(tmA, tmB, tmA, tmB, p);
}

// Two products of one shape in one grid (see UmmaParams::group_batch): the second product's operands come through
// their own tensor maps.  Whole tiles only, no row operation, beta = 0.
template <class T>
__global__ void __launch_bounds__(T::THREADS, 1)
umma_gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                         const UmmaParams p) {
  umma_gemm_core<T, false, 1, true>(tmA, tmB, tmA2, tmB2, p);
}

// Second pass of a split-K (or swapped-operand) GEMM: sums the `splits` raw partial results and applies
// the epilogue  v = alpha * sum + beta * C + bias ; Z = v ; C = act(v).  The partials are dense
// [batch, M, N], or [batch, N, M] when the GEMM ran with its operands swapped (`transposed`), in which
// case this pass also undoes the transposition.  One thread per output element, n fastest.
struct SplitKReduceParams {
  int M, N, batch, splits, transposed;
  const float* partial;
  long long partial_stride;
  float* C;
  float* Z;
  const float* bias;
  int ldc;
  long long strideC;
  float alpha, beta;
  int act;
  float act_alpha;
  OutMap omap;
};
static __global__ void splitk_reduce_kernel(const SplitKReduceParams p) {
  pdl_prologue();
  const long long per_batch = static_cast<long long>(p.M) * p.N;
  const long long total = per_batch * p.batch;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += stride) {
    const long long b = i / per_batch;
    const long long r = i - b * per_batch;
    const int m = static_cast<int>(r / p.N), n = static_cast<int>(r - static_cast<long long>(m) * p.N);
    const long long src = b * per_batch + (p.transposed ? static_cast<long long>(n) * p.M + m : r);
    float sum = 0.0f;
    for (int s = 0; s < p.splits; ++s) sum += p.partial[s * p.partial_stride + src];
    const long long off = p.omap.on ? out_offset(p.omap, static_cast<int>(b), m, n)
                                    : b * p.strideC + static_cast<long long>(m) * p.ldc + n;
    float v = p.alpha * sum;
    if (p.beta != 0.0f) v = fmaf(p.beta, p.C[off], v);
    if (p.bias) v += __ldg(p.bias + n);
    if (p.Z) p.Z[off] = v;
    p.C[off] = act_forward(p.act, v, p.act_alpha);
  }
}

// Same reduction for the swapped-operand plan, where the partials are [batch, N, M]: 32 x 32 tiles go
// through shared memory so that both the partial reads (m fastest) and the C accesses (n fastest) are
// coalesced.  Block = 32 x 8 threads; grid = (ceil(N/32), ceil(M/32), batch).
static __global__ void __launch_bounds__(256) splitk_reduce_transposed_kernel(const SplitKReduceParams p) {
  pdl_prologue();
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, m0 = blockIdx.y * 32, b = blockIdx.z;
  const long long per_batch = static_cast<long long>(p.M) * p.N;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    const int n = n0 + j, m = m0 + tx;
    float sum = 0.0f;
    if (n < p.N && m < p.M) {
      const long long src = b * per_batch + static_cast<long long>(n) * p.M + m;
      for (int s = 0; s < p.splits; ++s) sum += p.partial[s * p.partial_stride + src];
    }
    tile[j][tx] = sum;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int m = m0 + j, n = n0 + tx;
    if (m < p.M && n < p.N) {
      const long long off = p.omap.on ? out_offset(p.omap, b, m, n)
                                      : static_cast<long long>(b) * p.strideC + static_cast<long long>(m) * p.ldc + n;
      float v = p.alpha * tile[tx][j];
      if (p.beta != 0.0f) v = fmaf(p.beta, p.C[off], v);
      if (p.bias) v += __ldg(p.bias + n);
      if (p.Z) p.Z[off] = v;
      p.C[off] = act_forward(p.act, v, p.act_alpha);
    }
  }
}

// Second pass for the tiled workspace layout: sums the `splits` partial tiles of every tail tile and
// applies the epilogue.  Grid = (tail tiles, tile_rows / rows_per_block) with rows_per_block = 1024 / bn: a
// block of 256 threads covers 1024 elements of one tile, one float4 per thread, so that even a handful of
// tail tiles spreads over all SMs.
struct TailReduceParams {
  int M, N, tiles_m, tiles_n;   // tile grid as the GEMM kernel walked it (tile = tile_rows x bn)
  int tile_rows, bn, rows_per_block;
  int whole_tiles, tail, splits;
  const float* partial;
  long long tile_elems;         // tile_rows * bn
  float* C;
  float* Z;
  const float* bias;
  int ldc;
  long long strideC;
  float alpha, beta;
  int act;
  float act_alpha;
  int vec_ok;
  OutMap omap;
};
static __global__ void __launch_bounds__(256) tail_reduce_kernel(const TailReduceParams p) {
  pdl_prologue();
  int b, tm, tn;
  tile_coords(p.whole_tiles + blockIdx.x, p.tiles_m, p.tiles_n, b, tm, tn);
  const int r0 = blockIdx.y * p.rows_per_block;
  const int q_per_row = p.bn >> 2;
  const float* src = p.partial + static_cast<long long>(blockIdx.x) * p.tile_elems;
  const long long split_stride = static_cast<long long>(p.tail) * p.tile_elems;
  for (int i = threadIdx.x; i < p.rows_per_block * q_per_row; i += 256) {
    const int r = r0 + i / q_per_row;
    const int c = (i % q_per_row) << 2;
    const int row = tm * p.tile_rows + r, col = tn * p.bn + c;
    if (row >= p.M || col >= p.N) continue;
    const float* s0 = src + static_cast<long long>(r) * p.bn + c;
    float4 sum = *reinterpret_cast<const float4*>(s0);
#pragma unroll 4
    for (int s = 1; s < p.splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(s0 + s * split_stride);
      sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
    }
    const long long off = p.omap.on ? out_offset(p.omap, b, row, col)
                                    : static_cast<long long>(b) * p.strideC + static_cast<long long>(row) * p.ldc + col;
    float o[4] = {p.alpha * sum.x, p.alpha * sum.y, p.alpha * sum.z, p.alpha * sum.w};
    if (p.vec_ok && col + 4 <= p.N) {
      if (p.beta != 0.0f) {
        const float4 cin = *reinterpret_cast<const float4*>(p.C + off);
        o[0] = fmaf(p.beta, cin.x, o[0]); o[1] = fmaf(p.beta, cin.y, o[1]);
        o[2] = fmaf(p.beta, cin.z, o[2]); o[3] = fmaf(p.beta, cin.w, o[3]);
      }
      if (p.bias) {
        const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col));
        o[0] += bv.x; o[1] += bv.y; o[2] += bv.z; o[3] += bv.w;
      }
      if (p.Z) *reinterpret_cast<float4*>(p.Z + off) = make_float4(o[0], o[1], o[2], o[3]);
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = act_forward(p.act, o[e], p.act_alpha);
      *reinterpret_cast<float4*>(p.C + off) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      // a mapped result whose inner run d is not a multiple of 4: the four columns may lie in different runs
      for (int e = 0; e < 4 && col + e < p.N; ++e) {
        const long long oe = p.omap.on ? out_offset(p.omap, b, row, col + e) : off + e;
        float v = o[e];
        if (p.beta != 0.0f) v = fmaf(p.beta, p.C[oe], v);
        if (p.bias) v += __ldg(p.bias + col + e);
        if (p.Z) p.Z[oe] = v;
        p.C[oe] = act_forward(p.act, v, p.act_alpha);
      }
    }
  }
}

}  // namespace snb
