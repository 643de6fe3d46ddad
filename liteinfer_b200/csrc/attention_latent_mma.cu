// Latent attention on tensor cores (bfloat16): multi-query attention of up to 16 heads per row tile over the
// shared cache entries [latent (C) | rotated key part (R)], whose first C numbers are also the values
// (attention_latent.cu has the formulas and the SIMT kernel for every other size and for float32).
//
// A block of sixteen (or eight) warps takes MT row tiles of 16 rows, a row tile being ONE query's heads h0..h0+15, and walks
// the keys KT at a time (one bulk copy per entry into padded shared memory, a ring of stages behind mbarriers, the next
// tiles on their way while this one is used).  Per tile of keys:
//   1. scores: the units of 16 rows x 8 (or 16) keys are dealt to the warps, one unit a warp, or several warps a
//      unit, each then with a part of the (C + R) / 16 products and the parts added through shared memory; a
//      product is mma.sync m16n8k16 with the query rows (shared memory, ldmatrix) and the keys as they are stored
//      ([key][number] is the product's column-major operand).  Scale, causal mask, the unit's row maxima.
//   2. every row's new maximum from the units' maxima; probabilities, rounded to bfloat16, into shared memory;
//      the units' row sums.
//   3. values: warp w owns numbers [w * C / 16, (w + 1) * C / 16) of every row's accumulator (registers), rescales
//      them when a maximum moved and adds P V with the stored entries as the row-major operand (ldmatrix.trans).
// Three block barriers per tile (four where two warps share a unit).  Maxima are kept twice (the tile's old and new one) so that step 3 still finds the
// old one; sums are kept by the rows' own threads.  At the end the sink's term joins the denominator.
//
// Launches: sequences that bring one token run with MT = 1 (16 rows of 16 heads stream a sequence's entries
// once), either as two blocks of eight warps per SM (rounds of 32 keys, two stages) or as one block of sixteen
// warps (rounds of 64 keys from five stages of 32), their keys split over `num_splits`
// blocks whose partial results (normalised, with the logarithm of their denominators) a second kernel merges,
// sink included.  Sequences that bring more run with MT = 4, KT = 32 and three stages: four consecutive queries
// share every tile of keys.
#include "attention_mma.cuh"
#include "tcgen05.cuh"

namespace li {

struct LatentParams {
  const bf16* q_lat; long q_lat_head_stride; int q_lat_token_stride;
  const bf16* q_raw; int q_raw_token_stride, q_raw_head_stride, q_rot_off;
  bf16* out; long out_head_stride; int out_token_stride;
  const bf16* pool;
  const int* block_table; int table_stride;
  const int* query_start_loc; const int* context_lens;
  const int* seq_index;         // optional: batch row of each launched sequence (-1: a place of padding)
  const float* inv_freq; const float* sink;
  int heads, rot_dims, page_size, num_pages;
  float scale_log2;             // scale * log2(e)
  int num_splits;
  float* partial_out;           // [splits][heads][tokens][C] when num_splits > 1
  float* partial_lse;           // [splits][heads][tokens], in units of log2
  int tokens;
  int* error_flag;              // set to 31 if a wait for a tile of entries ever gave up (may be null)
  int window;                   // > 0: a query at position p reads the keys at p - window + 1 ... p
  float cs_scale;               // multiplies every cosine and sine of the query's rotation
};

// One entry (a contiguous run of bytes, 16-byte aligned at both ends) from global into shared memory by the copy
// engine; its bytes count towards the mbarrier's transaction.
__device__ __forceinline__ void bulk_load(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

constexpr int kMaxLatentWarps = 16;
constexpr int kTableCache = 2048;   // block-table entries a block keeps in shared memory (more are read in place)
constexpr int kPad = 8;         // bfloat16 of padding per shared-memory row: rows 16 bytes apart modulo 128

constexpr int kMaxStages = 6;

// KT: keys of one stage (one ring slot); SUB: stages used per round of the loop (KI = SUB * KT keys); NS: slots.
template <int C, int R, int MT, int KT, int SUB, int NS, int NW, int UK>
struct LatentSmem {
  static constexpr int KI = SUB * KT;
  static constexpr int D = C + R, LD = D + kPad, PLD = KI + kPad;
  static constexpr int kRows = MT * 16, kUnits = MT * (KI / UK);      // UK: keys of a score unit, 8 or 16
  static constexpr size_t q_bytes = (size_t)kRows * LD * 2;
  static constexpr size_t k_bytes = (size_t)KT * LD * 2;
  static constexpr size_t p_bytes = (size_t)kRows * PLD * 2;
  static constexpr int kSplitK = NW / kUnits;      // warps that share a unit, each with a part of the k-range
  static_assert(kSplitK * kUnits == NW && NW <= kMaxLatentWarps && NS > SUB && NS <= kMaxStages && KT % 16 == 0, "units must deal out evenly");
  static constexpr size_t f_floats = (size_t)kRows * (KI / 8) * 2 + kRows * 4;
  static constexpr size_t s_floats = (size_t)(kSplitK - 1) * kRows * KI;      // the other warps' partial scores
  static constexpr size_t total = q_bytes + NS * k_bytes + p_bytes + (f_floats + s_floats) * 4;
};

// Called by every warp: warp w brings keys [w * KT / NW, (w + 1) * KT / NW) of the stage, one lane a key.  The
// lane looks its key up in the block table; the warp's first lane arrives at the stage's mbarrier (which counts NW
// arrivals) and tells it how many bytes the warp's copies bring; then every visible entry is ONE bulk copy (no
// thread computes an address per 16 bytes, and no warp issues more than its share of the copies).  An entry that
// is not visible (behind the last query, or on a page given back) is written as zeros.
template <int C, int R, int KT, int NW>
__device__ __forceinline__ void load_key_tile(bf16* ks, unsigned bar, const LatentParams& p, const int* table,
                                              const int* cached, int cached_first, int cached_count, int key0,
                                              int limit) {
  constexpr int D = C + R, LD = D + kPad;
  constexpr unsigned kRowBytes = D * 2;
  constexpr int kPerWarp = KT / NW;
  static_assert(kPerWarp * NW == KT && kPerWarp >= 1 && kPerWarp <= 32, "the keys of a stage are dealt to the warps evenly");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = warp * kPerWarp + lane;            // the lane's key within the stage
  const bf16* src = nullptr;
  if (lane < kPerWarp) {
    const int kpos = key0 + row;
    if (kpos < limit) {
      // The block's part of the block table lies in shared memory (its first `cached_count` entries from
      // `cached_first` on); a look-up there does not hold the copies up for a trip to memory.
      const int block = kpos / p.page_size, at = block - cached_first;
      const int page = at < cached_count ? cached[at] : table[block];
      if (page >= 0 && page < p.num_pages) src = p.pool + ((size_t)page * p.page_size + kpos % p.page_size) * D;
    }
  }
  const int count = __reduce_add_sync(0xffffffffu, src != nullptr ? 1 : 0);
  if (lane < kPerWarp && !src) {
    bf16* dst = ks + row * LD;
    for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
    fence_async_shared();       // a later bulk copy into this row comes behind these stores
  }
  __syncwarp();
  if (lane == 0) mbar_expect_tx(bar, (unsigned)count * kRowBytes);      // the warp's arrival, and its bytes
  __syncwarp();
  if (src) bulk_load(smem_addr(ks + row * LD), src, kRowBytes, bar);
}

template <int C, int R, int MT, int KT, int SUB, int NS, int NW, int UK>
__global__ void __launch_bounds__(NW * 32, NW <= 8 ? 2 : 1)
latent_attention_mma_kernel(const LatentParams p) {
  using S = LatentSmem<C, R, MT, KT, SUB, NS, NW, UK>;
  static_assert(UK == 8 || UK == 16, "a score unit is one or two tiles of 8 keys");
  constexpr int kUnitTiles = UK / 8, kUnitsPerRow = S::KI / UK;
  constexpr int kLatentWarps = NW;
  constexpr int KI = S::KI;
  constexpr int D = S::D, LD = S::LD, PLD = S::PLD, kRows = S::kRows, kNTiles = KI / 8;
  constexpr int kOwnWarps = C / 8 < kLatentWarps ? C / 8 : kLatentWarps;   // warps that own a share of the accumulators
  constexpr int kOwn = C / kOwnWarps;            // numbers of the accumulator such a warp owns
  constexpr int kOwnTiles = kOwn / 8;
  constexpr int kSplitK = S::kSplitK;
  constexpr int kChunks32 = D / 32;              // the k-range in runs of 32 numbers, dealt to the warps of a unit
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* ks0 = reinterpret_cast<bf16*>(smem_raw + S::q_bytes);
  bf16* ps = reinterpret_cast<bf16*>(smem_raw + S::q_bytes + NS * S::k_bytes);
  float* unit_max = reinterpret_cast<float*>(smem_raw + S::q_bytes + NS * S::k_bytes + S::p_bytes);   // [kNTiles][kRows]
  float* unit_sum = unit_max + kNTiles * kRows;                                                       // [kNTiles][kRows]
  float* row_max = unit_sum + kNTiles * kRows;                                                        // [2][kRows]
  float* row_sum = row_max + 2 * kRows;                                                               // [kRows]
  float* row_inv = row_sum + kRows;                                                                   // [kRows]
  float* half_scores = row_inv + kRows;                                                               // [kSplitK - 1][kRows][KI]

  __shared__ __align__(8) unsigned long long stage_bars[kMaxStages];
  __shared__ int table_cache[kTableCache];
  grid_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const int split = p.num_splits > 1 ? blockIdx.x % p.num_splits : 0;
  // Blocks with the most keys first (a prompt's last queries): the short ones fill the end of the launch.
  const int tile_index = p.num_splits > 1 ? blockIdx.x / p.num_splits : gridDim.x - 1 - blockIdx.x;
  const int seq = p.seq_index ? p.seq_index[blockIdx.z] : blockIdx.z;
  if (seq < 0) return;
  const int q_begin = p.query_start_loc[seq], q_len = p.query_start_loc[seq + 1] - q_begin;
  const int query0 = tile_index * MT;
  if (query0 >= q_len) return;
  const int ctx = p.context_lens[seq];
  const int head0 = blockIdx.y * 16;
  const int* table = p.block_table + (size_t)seq * p.table_stride;
  const int first_pos = ctx - q_len + query0;                        // position of the block's first query
  const int last_pos = min(first_pos + MT - 1, ctx - 1);             // of its last one: the keys end there
  const int all_tiles = last_pos / KI + 1;                           // rounds of KI keys
  // With a window the first round is the one that holds the first key the block's first query still sees.
  const int tile_first = p.window > 0 ? max(first_pos - p.window + 1, 0) / KI : 0;
  const int per_split = (all_tiles - tile_first + p.num_splits - 1) / p.num_splits;
  const int tile_begin = tile_first + split * per_split, tile_end = min(all_tiles, tile_begin + per_split);

  const unsigned bars = smem_addr(stage_bars);
  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) mbar_init(bars + 8 * i, NW);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // The part of the block table that this block walks (an input of the step, not of a kernel ahead).
  const int cached_first = tile_begin * KI / p.page_size;
  const int cached_count = tile_begin < tile_end ? min(kTableCache, (min(tile_end * KI, last_pos + 1) - 1) / p.page_size + 1 - cached_first) : 0;
  for (int i = threadIdx.x; i < cached_count; i += kLatentWarps * 32) table_cache[i] = table[cached_first + i];
  __syncthreads();
  grid_dependency_wait();      // the entries of this step's tokens and the queries come from kernels ahead
  // Stage r of this block (r = 0, 1, ...) holds keys [(tile_begin * SUB + r) * KT, + KT), lies in slot r % NS and
  // turns that slot's barrier for the (r / NS)-th time.  A stage behind the last key is still "loaded": its rows are
  // written as zeros and its barrier turns, so the loop needs no special case for it.
  const int stages_total = (tile_end - tile_begin) * SUB;
  for (int r = 0; r < NS && r < stages_total; ++r)      // every slot filled before the first round
    load_key_tile<C, R, KT, NW>(ks0 + (size_t)r * KT * LD, bars + 8 * r, p, table, table_cache, cached_first, cached_count,
                                (tile_begin * SUB + r) * KT, last_pos + 1);

  // The query rows: row 16 * i + j is head head0 + j of query query0 + i; [absorbed query | rotated part].
  for (int i = threadIdx.x; i < kRows * (C / 8); i += kLatentWarps * 32) {
    const int row = i / (C / 8), chunk = i - row * (C / 8);
    const int query = query0 + row / 16, head = head0 + row % 16;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (query < q_len && head < p.heads)
      v = *reinterpret_cast<const uint4*>(p.q_lat + (size_t)head * p.q_lat_head_stride +
                                          (size_t)(q_begin + query) * p.q_lat_token_stride + chunk * 8);
    *reinterpret_cast<uint4*>(qs + row * LD + chunk * 8) = v;
  }
  {
    const int half = p.rot_dims / 2;
    for (int i = threadIdx.x; i < kRows * R; i += kLatentWarps * 32) {
      const int row = i / R, d = i - row * R;
      const int query = query0 + row / 16, head = head0 + row % 16;
      float v = 0.f;
      if (query < q_len && head < p.heads) {
        const bf16* qr = p.q_raw + (size_t)(q_begin + query) * p.q_raw_token_stride + (size_t)head * p.q_raw_head_stride + p.q_rot_off;
        if (d < p.rot_dims) {
          const int j = d < half ? d : d - half;
          const float angle = __fmul_rn((float)(first_pos + row / 16), p.inv_freq[j]);
          const float c = cosf(angle) * p.cs_scale, s = sinf(angle) * p.cs_scale;
          const float a = to_float(qr[j]), b = to_float(qr[j + half]);
          v = d < half ? rotate_lo(a, b, c, s) : rotate_hi(a, b, c, s);
        } else {
          v = to_float(qr[d]);
        }
      }
      qs[row * LD + C + d] = __float2bfloat16_rn(v);
    }
  }
  for (int i = threadIdx.x; i < kRows; i += kLatentWarps * 32) {
    row_max[i] = -INFINITY;
    row_max[kRows + i] = -INFINITY;
    row_sum[i] = 0.f;
  }

  float acc[MT][kOwnTiles][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int n = 0; n < kOwnTiles; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][n][e] = 0.f;

  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int it = tile - tile_begin;
    // This tile's entries have landed when its stage's barrier has turned (the next one's may be on their way).  A
    // wait that runs out raises the error flag; the block then stops, all of its threads together.
    bool landed = true;
#pragma unroll
    for (int j = 0; j < SUB; ++j) {
      const int r = it * SUB + j;
      landed = mbar_wait(bars + 8 * (r % NS), (unsigned)(r / NS) & 1, p.error_flag, 31) && landed;
    }
    if (__syncthreads_or(!landed)) break;
    // Every warp is past the round before this one (its probabilities and its stages may be overwritten).
    if (it > 0) {          // the slots that the round before this one used are free: fill them again
#pragma unroll
      for (int j = 0; j < SUB; ++j) {
        const int r = (it - 1) * SUB + j + NS;
        if (r < stages_total)
          load_key_tile<C, R, KT, NW>(ks0 + (size_t)(r % NS) * KT * LD, bars + 8 * (r % NS), p, table, table_cache,
                                      cached_first, cached_count, (tile_begin * SUB + r) * KT, last_pos + 1);
      }
    }
    const float* old_max = row_max + (it & 1) * kRows;
    float* new_max = row_max + ((it + 1) & 1) * kRows;
    const int key0 = tile * KI;

    // 1. scores: unit u = (row tile u / units per row, UK keys from UK * (u % units per row) on) belongs to warp u,
    //    or to warps u, u + units, ..., which then take a part of the k-range each and add their parts through
    //    shared memory.  A unit of 16 keys uses every fragment of the query rows for two tiles of keys.
    const int u = warp % S::kUnits, khalf = warp / S::kUnits;
    const int mt = u / kUnitsPerRow, nt0 = (u % kUnitsPerRow) * kUnitTiles;     // its first tile of 8 keys
    float sc[kUnitTiles][4];
#pragma unroll
    for (int j = 0; j < kUnitTiles; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
    {
      const bf16* qa = qs + (mt * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
      const bf16* slot = ks0 + (size_t)((it * SUB + nt0 * 8 / KT) % NS) * KT * LD;
      const int k_begin = (khalf * kChunks32 / kSplitK) * 32, k_end = ((khalf + 1) * kChunks32 / kSplitK) * 32;
      if (UK == 8) {
        const bf16* kb = slot + (nt0 * 8 % KT + (lane & 7)) * LD + (lane >> 3) * 8;
        // Four partial sums, each over every fourth k-step: the products of one sum wait for each other, not for
        // the other three's.
        float part[3][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 3
        for (int k0 = k_begin; k0 < k_end; k0 += 64) {
          unsigned a[4], a2[4], b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, kb + k0);          // keys nt0*8.., numbers k0..k0+31: two k-steps
          ldmatrix_x4(a[0], a[1], a[2], a[3], qa + k0);
          ldmatrix_x4(a2[0], a2[1], a2[2], a2[3], qa + k0 + 16);
          mma_bf16(sc[0], a, b0, b1);
          mma_bf16(part[0], a2, b2, b3);
          if (k0 + 32 < k_end) {
            ldmatrix_x4(b0, b1, b2, b3, kb + k0 + 32);
            ldmatrix_x4(a[0], a[1], a[2], a[3], qa + k0 + 32);
            ldmatrix_x4(a2[0], a2[1], a2[2], a2[3], qa + k0 + 48);
            mma_bf16(part[1], a, b0, b1);
            mma_bf16(part[2], a2, b2, b3);
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[0][e] += part[0][e] + part[1][e] + part[2][e];
      } else {
        // 16 keys x 16 numbers per fetch: (keys 0-7 | 8-15) x (numbers 0-7 | 8-15); even and odd k-steps add into
        // sums of their own, so four chains of products run side by side.
        const bf16* kb = slot + (nt0 * 8 % KT + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ((lane >> 3) & 1) * 8;
        float part[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
        for (int k0 = k_begin; k0 < k_end; k0 += 32) {
          unsigned a[4], a2[4], b0, b1, b2, b3, c0, c1, c2, c3;
          ldmatrix_x4(a[0], a[1], a[2], a[3], qa + k0);
          ldmatrix_x4(b0, b1, b2, b3, kb + k0);
          ldmatrix_x4(a2[0], a2[1], a2[2], a2[3], qa + k0 + 16);
          ldmatrix_x4(c0, c1, c2, c3, kb + k0 + 16);
          mma_bf16(sc[0], a, b0, b1);
          mma_bf16(sc[kUnitTiles - 1], a, b2, b3);
          mma_bf16(part[0], a2, c0, c1);
          mma_bf16(part[1], a2, c2, c3);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          sc[0][e] += part[0][e];
          sc[kUnitTiles - 1][e] += part[1][e];
        }
      }
    }
    if (kSplitK > 1) {
      float* lo = half_scores + (mt * 16 + g) * KI + nt0 * 8 + 2 * t4;
      if (khalf > 0) {
#pragma unroll
        for (int j = 0; j < kUnitTiles; ++j) {
          *reinterpret_cast<float2*>(lo + (khalf - 1) * kRows * KI + 8 * j) = make_float2(sc[j][0], sc[j][1]);
          *reinterpret_cast<float2*>(lo + (khalf - 1) * kRows * KI + 8 * KI + 8 * j) = make_float2(sc[j][2], sc[j][3]);
        }
      }
      __syncthreads();
      if (khalf == 0) {
#pragma unroll
        for (int part = 0; part < kSplitK - 1; ++part) {
#pragma unroll
          for (int j = 0; j < kUnitTiles; ++j) {
            const float2 x = *reinterpret_cast<const float2*>(lo + part * kRows * KI + 8 * j);
            const float2 y = *reinterpret_cast<const float2*>(lo + part * kRows * KI + 8 * KI + 8 * j);
            sc[j][0] += x.x; sc[j][1] += x.y; sc[j][2] += y.x; sc[j][3] += y.y;
          }
        }
      }
    }
    if (khalf == 0) {
      // Scale, mask (key j is visible to the query at position pos iff j <= pos), and the row maxima per tile of 8 keys.
      const int pos = first_pos + mt;
#pragma unroll
      for (int j = 0; j < kUnitTiles; ++j) {
        const int nt = nt0 + j;
        const int kcol = key0 + nt * 8 + 2 * t4;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kcol + (e & 1);
          sc[j][e] = (key <= pos && (p.window <= 0 || key > pos - p.window)) ? sc[j][e] * p.scale_log2 : -INFINITY;
        }
        float m_lo = fmaxf(sc[j][0], sc[j][1]), m_hi = fmaxf(sc[j][2], sc[j][3]);
        m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 1));
        m_lo = fmaxf(m_lo, __shfl_xor_sync(0xffffffffu, m_lo, 2));
        m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 1));
        m_hi = fmaxf(m_hi, __shfl_xor_sync(0xffffffffu, m_hi, 2));
        if (t4 == 0) {
          unit_max[nt * kRows + mt * 16 + g] = m_lo;
          unit_max[nt * kRows + mt * 16 + g + 8] = m_hi;
        }
      }
    }
    __syncthreads();

    // 2. the rows' new maxima (their own threads store them), probabilities into shared memory, the tiles' sums.
    if (threadIdx.x < kRows) {
      float m = old_max[threadIdx.x];
#pragma unroll
      for (int n = 0; n < kNTiles; ++n) m = fmaxf(m, unit_max[n * kRows + threadIdx.x]);
      new_max[threadIdx.x] = m;
    }
    if (khalf == 0) {
      const int r_lo = mt * 16 + g, r_hi = r_lo + 8;
      float m_lo = old_max[r_lo], m_hi = old_max[r_hi];
#pragma unroll
      for (int n = 0; n < kNTiles; ++n) {
        m_lo = fmaxf(m_lo, unit_max[n * kRows + r_lo]);
        m_hi = fmaxf(m_hi, unit_max[n * kRows + r_hi]);
      }
#pragma unroll
      for (int j = 0; j < kUnitTiles; ++j) {
        const int nt = nt0 + j;
        const float p0 = m_lo == -INFINITY ? 0.f : fast_exp2(sc[j][0] - m_lo);
        const float p1 = m_lo == -INFINITY ? 0.f : fast_exp2(sc[j][1] - m_lo);
        const float p2 = m_hi == -INFINITY ? 0.f : fast_exp2(sc[j][2] - m_hi);
        const float p3 = m_hi == -INFINITY ? 0.f : fast_exp2(sc[j][3] - m_hi);
        *reinterpret_cast<__nv_bfloat162*>(ps + r_lo * PLD + nt * 8 + 2 * t4) = __floats2bfloat162_rn(p0, p1);
        *reinterpret_cast<__nv_bfloat162*>(ps + r_hi * PLD + nt * 8 + 2 * t4) = __floats2bfloat162_rn(p2, p3);
        float s_lo = p0 + p1, s_hi = p2 + p3;
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1);
        s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1);
        s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
        if (t4 == 0) {
          unit_sum[nt * kRows + r_lo] = s_lo;
          unit_sum[nt * kRows + r_hi] = s_hi;
        }
      }
    }
    __syncthreads();

    // 3. the rows' sums (their own threads), and every warp's share of the accumulators.
    if (threadIdx.x < kRows) {
      const float m_old = old_max[threadIdx.x], m_new = new_max[threadIdx.x];
      float s = 0.f;
#pragma unroll
      for (int n = 0; n < kNTiles; ++n) s += unit_sum[n * kRows + threadIdx.x];
      const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_old - m_new);
      row_sum[threadIdx.x] = row_sum[threadIdx.x] * alpha + s;
    }
    if (warp < kOwnWarps) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int r_lo = mt * 16 + g, r_hi = r_lo + 8;
        const float n_lo = new_max[r_lo], n_hi = new_max[r_hi];
        const float a_lo = n_lo == -INFINITY ? 1.f : fast_exp2(old_max[r_lo] - n_lo);
        const float a_hi = n_hi == -INFINITY ? 1.f : fast_exp2(old_max[r_hi] - n_hi);
        if (a_lo != 1.f || a_hi != 1.f) {
#pragma unroll
          for (int n = 0; n < kOwnTiles; ++n) {
            acc[mt][n][0] *= a_lo; acc[mt][n][1] *= a_lo;
            acc[mt][n][2] *= a_hi; acc[mt][n][3] *= a_hi;
          }
        }
      }
      // The entries' fragments are fetched once per 16 keys and serve every row tile.
#pragma unroll
      for (int k0 = 0; k0 < KI; k0 += 16) {
        const bf16* vb = ks0 + (size_t)((it * SUB + k0 / KT) % NS) * KT * LD +
                         (k0 % KT + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + warp * kOwn + (lane >> 4) * 8;
        unsigned vf[(kOwnTiles + 1) / 2][4];
#pragma unroll
        for (int n = 0; n < kOwnTiles; n += 2)
          ldmatrix_x4_trans(vf[n / 2][0], vf[n / 2][1], vf[n / 2][2], vf[n / 2][3], vb + n * 8);   // two 8-wide tiles
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          unsigned a[4];
          ldmatrix_x4(a[0], a[1], a[2], a[3], ps + (mt * 16 + (lane & 15)) * PLD + (lane >> 4) * 8 + k0);
#pragma unroll
          for (int n = 0; n < kOwnTiles; n += 2) {
            mma_bf16(acc[mt][n], a, vf[n / 2][0], vf[n / 2][1]);
            if (n + 1 < kOwnTiles) mma_bf16(acc[mt][n + 1], a, vf[n / 2][2], vf[n / 2][3]);
          }
        }
      }
    }
  }
  __syncthreads();
  // The end: denominators (with the sink's term where this block sees all keys), then the rows leave.
  const int final_buf = ((tile_end > tile_begin ? tile_end - tile_begin : 0) & 1) * kRows;   // where the last tile left the maxima
  if (threadIdx.x < kRows) {
    const int head = head0 + threadIdx.x % 16;
    float m = row_max[final_buf + threadIdx.x], l = row_sum[threadIdx.x];
    if (p.num_splits <= 1) {
      if (p.sink && head < p.heads) {
        const float sk = p.sink[head] * kLog2e;
        const float m_new = fmaxf(m, sk);
        const float alpha = m == -INFINITY ? 0.f : fast_exp2(m - m_new);
        l = l * alpha + fast_exp2(sk - m_new);
        row_inv[threadIdx.x] = l > 0.f ? alpha / l : 0.f;
      } else {
        row_inv[threadIdx.x] = l > 0.f ? 1.f / l : 0.f;
      }
    } else {
      row_inv[threadIdx.x] = l > 0.f ? 1.f / l : 0.f;
      const int query = query0 + threadIdx.x / 16;
      if (query < q_len && head < p.heads)
        p.partial_lse[((size_t)split * p.heads + head) * p.tokens + q_begin + query] = l > 0.f ? m + log2f(l) : -INFINITY;
    }
  }
  __syncthreads();
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int query = query0 + mt;
    if (query >= q_len || warp >= kOwnWarps) continue;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int head = head0 + g + hh * 8;
      if (head >= p.heads) continue;
      const float inv = row_inv[mt * 16 + g + hh * 8];
#pragma unroll
      for (int n = 0; n < kOwnTiles; ++n) {
        const int col = warp * kOwn + n * 8 + 2 * t4;
        const float x = acc[mt][n][2 * hh] * inv, y = acc[mt][n][2 * hh + 1] * inv;
        if (p.num_splits <= 1) {
          bf16* o = p.out + (size_t)head * p.out_head_stride + (size_t)(q_begin + query) * p.out_token_stride + col;
          *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(x, y);
        } else {
          float* o = p.partial_out + (((size_t)split * p.heads + head) * p.tokens + q_begin + query) * C + col;
          *reinterpret_cast<float2*>(o) = make_float2(x, y);
        }
      }
    }
  }
}

// The splits of a (token, head) row merged: out = sum_s w_s O_s / (sum_s w_s + the sink's term), w_s = 2^(lse_s - max).
// The weights are worked out once per block; a thread adds up its numbers kBatch splits at a time, all their loads
// on their way at once.
constexpr int kMaxSplits = 32;
template <int kBatch>      // partial rows a thread has on their way at once: few for few splits (fewer registers)
__global__ void latent_merge_kernel(const float* __restrict__ partial_out, const float* __restrict__ partial_lse,
                                    const int* __restrict__ seq_index, const int* __restrict__ query_start_loc,
                                    bf16* __restrict__ out, long out_head_stride,
                                    int out_token_stride, const float* __restrict__ sink, int heads, int tokens,
                                    int C, int num_splits) {
  __shared__ float weight[kMaxSplits];
  // What the step itself brings (the sequence list, the tokens' places, the sinks) is read while the kernel ahead
  // still runs; its partial results only behind the wait.
  const int seq = seq_index ? seq_index[blockIdx.x] : blockIdx.x;
  const int head = blockIdx.y;
  const int token = seq < 0 ? 0 : query_start_loc[seq];         // the sequence's one token
  const float sk = sink ? sink[head] * kLog2e : -INFINITY;
  grid_dependency_wait();
  grid_launch_dependents();
  if (seq < 0) return;                            // a place of padding
  // A thread's first partial rows are on their way while the first warp works out the weights.
  float4 x[kBatch];
  const int d0 = threadIdx.x * 4;
  auto part = [&](int s, int d) {
    return *reinterpret_cast<const float4*>(partial_out + (((size_t)s * heads + head) * tokens + token) * C + d);
  };
  if (d0 < C) {
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (j < num_splits) x[j] = part(j, d0);
  }
  if (threadIdx.x < 32) {
    const float lse = (int)threadIdx.x < num_splits
                          ? partial_lse[((size_t)threadIdx.x * heads + head) * tokens + token] : -INFINITY;
    float m = fmaxf(lse, sk);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float w = m == -INFINITY ? 0.f : exp2f(lse - m);
    float denom = w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    if (sink && m != -INFINITY) denom += exp2f(sk - m);
    weight[threadIdx.x] = denom > 0.f ? w / denom : 0.f;
  }
  __syncthreads();
  for (int d = d0; d < C; d += blockDim.x * 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int base = 0; base < num_splits; base += kBatch) {
      if (d != d0 || base != 0) {
#pragma unroll
        for (int j = 0; j < kBatch; ++j)
          if (base + j < num_splits) x[j] = part(base + j, d);
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (base + j < num_splits) {
          const float w = weight[base + j];
          v.x = fmaf(w, x[j].x, v.x); v.y = fmaf(w, x[j].y, v.y); v.z = fmaf(w, x[j].z, v.z); v.w = fmaf(w, x[j].w, v.w);
        }
      }
    }
    bf16* o = out + (size_t)head * out_head_stride + (size_t)token * out_token_stride + d;
    *reinterpret_cast<__nv_bfloat162*>(o) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(o + 2) = __floats2bfloat162_rn(v.z, v.w);
  }
}

template <int C, int R, int MT, int KT, int SUB, int NS, int NW, int UK>
int launch_latent(const LatentParams& p, int num_seqs, int row_tiles, cudaStream_t stream) {
  using S = LatentSmem<C, R, MT, KT, SUB, NS, NW, UK>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<C, R, MT, KT, SUB, NS, NW, UK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::total);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const dim3 grid(row_tiles * (p.num_splits > 1 ? p.num_splits : 1), (p.heads + 15) / 16, num_seqs);
  return (int)launch_pdl(row_tiles * MT, latent_attention_mma_kernel<C, R, MT, KT, SUB, NS, NW, UK>, grid, dim3(NW * 32),
                         S::total, stream, p);
}

template <int C, int R>
int launch_latent_sizes(const LatentParams& p, int num_seqs, int max_q_len, int two_blocks, cudaStream_t stream) {
  // Stages of entries on their way: as many as shared memory holds beside the query rows.
  if (max_q_len == 1) {
    // Two blocks of eight warps per SM (rounds of 32 keys, two stages each): while one block stands at a barrier
    // the other works.  Or one block of sixteen warps (rounds of 64 keys from five stages of 32): fewer, longer
    // blocks, which a narrow batch with many splits does a little better with.
    if (two_blocks) return launch_latent<C, R, 1, 32, 1, 2, 8, 8>(p, num_seqs, 1, stream);
    return launch_latent<C, R, 1, 32, 2, 5, 16, 8>(p, num_seqs, 1, stream);
  }
  return launch_latent<C, R, 4, 32, 1, 3, 16, 16>(p, num_seqs, (max_q_len + 3) / 4, stream);
}

}  // namespace li

using namespace li;

LI_EXPORT int li_latent_attention_mma_supports(int kv_rank, int rot_dim, int rot_dims) {
  const bool sizes = (kv_rank == 64 && rot_dim == 32) || (kv_rank == 128 && (rot_dim == 32 || rot_dim == 64)) ||
                     (kv_rank == 256 && rot_dim == 64) || (kv_rank == 512 && rot_dim == 64);
  return sizes && rot_dims >= 0 && rot_dims <= rot_dim && (rot_dims & 1) == 0;
}

// As li_latent_attention (attention_latent.cu), bfloat16 only, for the sizes `..._supports` names.  seq_index
// [num_seqs] or null: the batch rows to run (-1: none); max_q_len 1 runs the single-token form, whose keys
// `num_splits` blocks share (partial_out [splits, heads, tokens, kv_rank] and partial_lse [splits, heads, tokens]
// float; `tokens`: the step's token rows; `two_blocks`: the single-token form as two blocks of eight warps per SM).  error_flag (device int, zero; may be null): set to 31 if a wait for a
// tile of entries ever gave up.  window > 0: a query sees the newest `window` keys up to its own; cos_sin_scale
// multiplies every cosine and sine of the query's rotation.
LI_EXPORT int li_latent_attention_mma(const void* q_lat, long q_lat_head_stride, int q_lat_token_stride,
                                      const void* q_raw, int q_raw_token_stride, int q_raw_head_stride, int q_rot_off,
                                      void* out, long out_head_stride, int out_token_stride, const void* pool,
                                      const int* block_table, int table_stride, const int* query_start_loc,
                                      const int* context_lens, const int* seq_index, const float* inv_freq,
                                      const float* sink, int num_seqs, int max_q_len, int heads, int kv_rank,
                                      int rot_dim, int rot_dims, int page_size, int num_pages, float scale,
                                      int num_splits, float* partial_out, float* partial_lse, int tokens,
                                      int two_blocks, int* error_flag, int window, float cos_sin_scale,
                                      cudaStream_t stream) {
  if (num_seqs == 0 || max_q_len == 0) return 0;
  if (!li_latent_attention_mma_supports(kv_rank, rot_dim, rot_dims) || num_seqs > 65535) return LI_ERR_UNSUPPORTED;
  if (!aligned16(q_lat) || !aligned16(pool) || (q_lat_token_stride % 8) || (q_lat_head_stride % 8) || (out_token_stride % 2) ||
      (out_head_stride % 2))
    return LI_ERR_ALIGNMENT;
  if (max_q_len != 1) num_splits = 1;
  if (num_splits > kMaxSplits) num_splits = kMaxSplits;
  if (num_splits > 1 && (!partial_out || !partial_lse)) return LI_ERR_UNSUPPORTED;
  LatentParams p;
  p.q_lat = (const bf16*)q_lat; p.q_lat_head_stride = q_lat_head_stride; p.q_lat_token_stride = q_lat_token_stride;
  p.q_raw = (const bf16*)q_raw; p.q_raw_token_stride = q_raw_token_stride; p.q_raw_head_stride = q_raw_head_stride;
  p.q_rot_off = q_rot_off;
  p.out = (bf16*)out; p.out_head_stride = out_head_stride; p.out_token_stride = out_token_stride;
  p.pool = (const bf16*)pool; p.block_table = block_table; p.table_stride = table_stride;
  p.query_start_loc = query_start_loc; p.context_lens = context_lens; p.seq_index = seq_index;
  p.inv_freq = inv_freq; p.sink = sink; p.heads = heads; p.rot_dims = rot_dims; p.page_size = page_size;
  p.num_pages = num_pages; p.scale_log2 = scale * kLog2e; p.num_splits = num_splits < 1 ? 1 : num_splits;
  p.partial_out = partial_out; p.partial_lse = partial_lse; p.tokens = tokens; p.error_flag = error_flag;
  p.window = window; p.cs_scale = cos_sin_scale;
  int code;
  if (kv_rank == 64) code = launch_latent_sizes<64, 32>(p, num_seqs, max_q_len, two_blocks, stream);
  else if (kv_rank == 128 && rot_dim == 32) code = launch_latent_sizes<128, 32>(p, num_seqs, max_q_len, two_blocks, stream);
  else if (kv_rank == 128) code = launch_latent_sizes<128, 64>(p, num_seqs, max_q_len, two_blocks, stream);
  else if (kv_rank == 256) code = launch_latent_sizes<256, 64>(p, num_seqs, max_q_len, two_blocks, stream);
  else code = launch_latent_sizes<512, 64>(p, num_seqs, max_q_len, two_blocks, stream);
  if (code != 0 || p.num_splits <= 1) return code;
  return (int)launch_pdl(num_seqs, p.num_splits <= 4 ? latent_merge_kernel<4> : latent_merge_kernel<16>, dim3(num_seqs, heads),
                         dim3(128), 0, stream, (const float*)partial_out, (const float*)partial_lse, seq_index,
                         query_start_loc, (bf16*)out, out_head_stride, out_token_stride, sink, heads, tokens, kv_rank,
                         p.num_splits);
}
