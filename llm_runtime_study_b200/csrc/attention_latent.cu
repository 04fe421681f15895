// bfloat16 tensor-core attention of many query heads over ONE shared row per token whose leading columns are also
// the value (latent attention with the up-projections moved to the query's side), built once per pair of sizes
// (-DLATENT_RANK=<value columns> -DLATENT_ROT=<further key columns>, both multiples of 16).
//
// A CTA takes up to BM = 64 rows: consecutive query tokens of one request times the heads of one group of at most 64
// heads.  Keys are streamed in tiles of 32 rows through shared memory (cp.async, two stages) from the request's pages.
// Eight warps: warp w owns rows 16 (w & 3) .. + 15 and the value columns of half (w >> 2); both warps of a row group
// form the same scores S = Q K^T (mma.sync m16n8k16, float accumulation), run the same online softmax in float32, round
// P to bfloat16 and multiply it with their half of the value columns, read transposed out of the key tile.
// Key t is visible to a query at position p iff t <= p and (window == 0 or t > p - window).
#include "common.cuh"
#include "mma.cuh"

#if !defined(LATENT_RANK) || !defined(LATENT_ROT)
#error "compile with -DLATENT_RANK=<value columns> -DLATENT_ROT=<further key columns>"
#endif
static_assert(LATENT_RANK % 16 == 0 && LATENT_RANK >= 16 && LATENT_RANK <= 512, "the value width must be 16..512 in steps of 16");
static_assert(LATENT_ROT % 16 == 0 && LATENT_ROT >= 0, "the further key columns come in steps of 16");

namespace b200 {

using bf16 = __nv_bfloat16;
constexpr int DV = LATENT_RANK, DK = LATENT_RANK + LATENT_ROT;
constexpr int BM = 64, BN = 32, NT = 256;
constexpr int LDS = DK + 8;                 // padded row: ldmatrix rows fall into different banks
constexpr int KSTEPS = DK / 16;
constexpr int DVH = DV / 2;                 // value columns of one warp
constexpr int OTILES = DVH / 8;
constexpr int kSmemBytes = (BM + 2 * BN) * LDS * 2;

struct LatentParams {
  const bf16* q;            // [n, heads, DK]
  const bf16* pool;         // [pages, page_size, DK]
  bf16* out;                // [n, heads, DV]
  const int* positions;     // [n]
  const int* block_table;   // [entries, table_stride]
  const int* tile_entry;    // per tile: entry, first token (index into the batch's rows), tokens
  const int* tile_start;
  const int* tile_count;
  int table_stride, page_size, heads, group_heads, tokens_per_tile, window;
  float scale_log2;
  // a tile's keys cut into `splits` parts (single tokens only): CTA z takes its share of the key tiles and leaves
  // (maximum, sum) and the unnormalised output of row token * heads + head in scratch memory for the merge kernel
  int splits;
  float* part_o;    // [rows][splits][DV]
  float* part_ml;   // [rows][splits][2]
};

__device__ __forceinline__ void load_key_tile(bf16* ks, const LatentParams& p, const int* table, int t0, int lo, int hi) {
  constexpr int CH = DK / 8;
  for (int c = threadIdx.x; c < BN * CH; c += NT) {
    const int r = c / CH, ch = c - r * CH;
    const int t = t0 + r;
    const bf16* src = p.pool;
    int bytes = 0;
    if (t >= lo && t <= hi) {
      const int page = table[t / p.page_size];
      if (page >= 0) {
        src = p.pool + (static_cast<size_t>(page) * p.page_size + t % p.page_size) * DK + ch * 8;
        bytes = 16;
      }
    }
    cp_async_16(ks + r * LDS + ch * 8, src, bytes);
  }
}

__global__ void __launch_bounds__(NT, 1)
latent_attention_kernel(const LatentParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* ks = qs + BM * LDS;
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x, hgroup = blockIdx.y;
  const int entry = p.tile_entry[tile], start = p.tile_start[tile], count = p.tile_count[tile];
  const int hg = min(p.group_heads, p.heads - hgroup * p.group_heads);
  const int* table = p.block_table + static_cast<size_t>(entry) * p.table_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rg = warp & 3, half = warp >> 2;

  // the rows of this thread: r0 = 16 rg + lane / 4 and r0 + 8; row r is token r / hg, head r % hg of the tile
  int pos[2], row_token[2], row_head[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rg * 16 + (lane >> 2) + i * 8;
    const int tl = r / hg, hl = r - tl * hg;
    const bool valid = tl < count && tl < p.tokens_per_tile;
    row_token[i] = valid ? start + tl : -1;
    row_head[i] = hgroup * p.group_heads + hl;
    pos[i] = valid ? p.positions[start + tl] : -1;
  }
  const int p_first = p.positions[start], p_last = p.positions[start + count - 1];
  const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0, hi = p_last;

  // Q tile
  {
    constexpr int CH = DK / 8;
    for (int c = threadIdx.x; c < BM * CH; c += NT) {
      const int r = c / CH, ch = c - r * CH;
      const int tl = r / hg, hl = r - tl * hg;
      const bool valid = tl < count && tl < p.tokens_per_tile;
      const bf16* src = valid ? p.q + (static_cast<size_t>(start + tl) * p.heads + hgroup * p.group_heads + hl) * DK + ch * 8 : p.q;
      cp_async_16(qs + r * LDS + ch * 8, src, valid ? 16 : 0);
    }
  }
  int t_begin = (lo / BN) * BN;
  int tiles = hi >= t_begin ? (hi - t_begin) / BN + 1 : 0;
  if (p.splits > 1) {          // this CTA's share of the key tiles
    const int per = (tiles + p.splits - 1) / p.splits;
    const int first_tile = min(tiles, static_cast<int>(blockIdx.z) * per);
    tiles = min(tiles - first_tile, per);
    t_begin += first_tile * BN;
  }
  if (tiles > 0) load_key_tile(ks, p, table, t_begin, lo, hi);
  cp_async_commit();

  float o[OTILES][4];
#pragma unroll
  for (int j = 0; j < OTILES; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int kt = 0; kt < tiles; ++kt) {
    const int t0 = t_begin + kt * BN;
    bf16* kcur = ks + (kt & 1) * BN * LDS;
    if (kt + 1 < tiles) load_key_tile(ks + ((kt + 1) & 1) * BN * LDS, p, table, t0 + BN, lo, hi);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    // S = Q K^T for this warp's 16 rows and the tile's 32 keys
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll 4
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t a[4], b[2][4];
      ldmatrix_x4(a, qs + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        ldmatrix_x4(b[j], kcur + (j * 16 + (lane & 7) + (lane >> 4) * 8) * LDS + kk * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) mma_bf16(s[j], a, b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
    }
    // mask, online softmax (base 2)
    float m_new[2] = {m[0], m[1]};
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int t = t0 + j * 8 + (lane & 3) * 2 + (e & 1);
        const bool seen = pos[i] >= 0 && t <= pos[i] && (p.window == 0 || t > pos[i] - p.window);
        s[j][e] = seen ? s[j][e] * p.scale_log2 : -INFINITY;
        m_new[i] = fmaxf(m_new[i], s[j][e]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
    }
    float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float base = m_new[i] == -INFINITY ? 0.f : m_new[i];
      corr[i] = exp2f(m[i] - base);        // m = -inf: 0
      m[i] = m_new[i];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = exp2f(s[j][i * 2 + e] - base);
          s[j][i * 2 + e] = pv;
          sum[i] += pv;
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
      l[i] = l[i] * corr[i] + sum[i];
    }
#pragma unroll
    for (int j = 0; j < OTILES; ++j) {
      o[j][0] *= corr[0]; o[j][1] *= corr[0];
      o[j][2] *= corr[1]; o[j][3] *= corr[1];
    }
    // O += P V, V = this warp's half of the leading columns of the key rows
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int j = 0; j < OTILES; j += 2) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, kcur + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + half * DVH + j * 8 + (lane >> 4) * 8);
        mma_bf16(o[j], a, b[0], b[1]);
        if (j + 1 < OTILES) mma_bf16(o[j + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  if (p.splits > 1) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      if (row_token[i] < 0 || row_head[i] >= p.heads) continue;
      const size_t slot = (static_cast<size_t>(row_token[i]) * p.heads + row_head[i]) * p.splits + blockIdx.z;
      if (half == 0 && (lane & 3) == 0) {
        p.part_ml[slot * 2] = m[i];
        p.part_ml[slot * 2 + 1] = l[i];
      }
      float* dst = p.part_o + slot * DV + half * DVH + (lane & 3) * 2;
#pragma unroll
      for (int j = 0; j < OTILES; ++j) *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][i * 2], o[j][i * 2 + 1]);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (row_token[i] < 0 || row_head[i] >= p.heads || (rg * 16 + (lane >> 2) + i * 8) / hg >= p.tokens_per_tile) continue;
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
    bf16* dst = p.out + (static_cast<size_t>(row_token[i]) * p.heads + row_head[i]) * DV + half * DVH + (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < OTILES; ++j)
      *reinterpret_cast<__nv_bfloat162*>(dst + j * 8) = __floats2bfloat162_rn(o[j][i * 2] * inv, o[j][i * 2 + 1] * inv);
  }
}

// out[row] = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z over the parts of a row's keys, M the largest maximum.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out, int splits) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;
  float top = -INFINITY;
  for (int z = 0; z < splits; ++z) top = fmaxf(top, part_ml[(row * splits + z) * 2]);
  float total = 0.f;
  for (int z = 0; z < splits; ++z) {
    const float mz = part_ml[(row * splits + z) * 2];
    total += mz == -INFINITY ? 0.f : exp2f(mz - top) * part_ml[(row * splits + z) * 2 + 1];
  }
  const float inv = total > 0.f ? 1.f / total : 0.f;
  for (int c = threadIdx.x; c < DV; c += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float mz = part_ml[(row * splits + z) * 2];
      if (mz != -INFINITY) acc = fmaf(exp2f(mz - top), part_o[(row * splits + z) * DV + c], acc);
    }
    out[row * DV + c] = __float2bfloat16_rn(acc * inv);
  }
}

DeviceOnce latent_once;

}  // namespace b200

extern "C" int b200_attention_latent_rank() { return b200::DV; }
extern "C" int b200_attention_latent_rot() { return LATENT_ROT; }

// q [n, heads, DK], pool [pages, page_size, DK], out [n, heads, DV]; tiles: (entry, first row, rows) of consecutive
// tokens of one entry, at most tokens_per_tile = max(1, 64 / heads) each.  splits > 1 (every tile is token t alone, tile t):
// the keys of a token are cut into that many parts, merged by a second launch; scratch holds splits * (DV + 2) floats a row.
extern "C" int b200_attention_latent_bf16(const void* q, const void* pool, void* out, const int* positions, const int* block_table,
                                          int table_stride, int page_size, int heads, float scale, int window, const int* tile_entry,
                                          const int* tile_start, const int* tile_count, int num_tiles, int splits, float* scratch,
                                          long scratch_floats, cudaStream_t stream) {
  using namespace b200;
  if (num_tiles <= 0) return 0;
  if (heads <= 0 || page_size <= 0 || window < 0 || splits < 1 || splits > 64) return B200_ERR_BAD_SIZE;
  // parts only for single tokens (one tile a token): the scratch rows are token * heads + head
  if (splits > 1 && (scratch == nullptr || scratch_floats < static_cast<long>(num_tiles) * heads * splits * (DV + 2))) return 10004;
  const int status = configure_once(latent_once, latent_attention_kernel, kSmemBytes);
  if (status != 0) return status;
  LatentParams p{};
  p.q = static_cast<const bf16*>(q);
  p.pool = static_cast<const bf16*>(pool);
  p.out = static_cast<bf16*>(out);
  p.positions = positions;
  p.block_table = block_table;
  p.tile_entry = tile_entry;
  p.tile_start = tile_start;
  p.tile_count = tile_count;
  p.table_stride = table_stride;
  p.page_size = page_size;
  p.heads = heads;
  p.group_heads = heads < BM ? heads : BM;
  p.tokens_per_tile = BM / p.group_heads;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.splits = splits;
  if (splits > 1) {
    p.tokens_per_tile = 1;
    p.part_o = scratch;
    p.part_ml = scratch + static_cast<size_t>(num_tiles) * heads * splits * DV;
  }
  dim3 grid(num_tiles, (heads + p.group_heads - 1) / p.group_heads, splits);
  if (grid.y > 65535) return B200_ERR_TOO_LARGE;
  launch(latent_attention_kernel, grid, dim3(NT), kSmemBytes, stream, p);
  if (splits > 1) launch(latent_merge_kernel, dim3(num_tiles * heads), dim3(128), 0, stream, p.part_o, p.part_ml, p.out, splits);
  return launch_status();
}
