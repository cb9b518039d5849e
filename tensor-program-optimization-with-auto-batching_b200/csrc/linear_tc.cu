// Weight-streaming projection kernel on the 5th-generation tensor cores (tcgen05 + TMEM), fed by
// TMA.  y[T,out] = x[T,in] W[out,in]^T with T small (decode) or tiled (prefill): the weight tile
// is the 128-row M operand, the token rows are the N operand ("swap-AB"), so a 128 x BN fp32
// accumulator lives in BN TMEM columns and one thread issues all MMAs.
//
// Persistent and warp-specialised:
//   * one CTA per SM (grid <= SM count), 224 threads: warp 0 = weight producer, warp 1 = MMA issuer
//     (one thread each), warps 2..5 = epilogue (one TMEM lane = one output row per thread), warp 6 =
//     token-tile producer and builder of the LoRA operands (at prompt sizes the epilogue warps build the
//     cached operands instead, while the tile's MMAs run).  Weights stream from HBM through a ring of
//     up to 10 x 16 KB stages (one bulk copy per pre-tiled stage); token tiles come from L2 through
//     their own shallow ring;
//   * decode sizes (stream-K): the iteration space (tile, k-block) -- tiles = row tiles x token tiles,
//     k-blocks of 64 -- is cut into equal contiguous ranges, one per CTA, so every SM streams the same
//     number of bytes whatever the shape; a range covers a tail of one tile, whole tiles, and a head of
//     another.  Prefill sizes: whole tiles of 128 or 256 tokens only, dealt in token-tile groups whose CTAs walk
//     the row tiles in lockstep lanes (see wave_tile);
//   * two TMEM accumulators: the epilogue of one segment overlaps the MMAs of the next, and the
//     shared-memory ring keeps filling across segment boundaries;
//   * a tile whose k-blocks are spread over several CTAs is finished by the CTA that holds its FIRST
//     k-blocks (it reaches them last, at the end of its range): the other contributors write their fp32
//     partial tile to scratch and bump the tile's counter; the finisher waits (bounded) for the counter,
//     sums the partials in CTA order (deterministic) while its own last MMAs still run, and runs the
//     epilogue (SiLU*up, staging, TMA store).  The tile's LoRA stages run in the finisher as well.
//
// Every wait is bounded; on expiry the CTA records a code in the status word at the start of the
// scratch buffer, stops issuing work, and leaves after freeing its TMEM.
#include <stdlib.h>

#include <atomic>

#include "linear.cuh"
#include "tc_ptx.cuh"

namespace mlora {
namespace {

constexpr int BM = 128;            // weight rows per tile (MMA M)
constexpr int kThreads = 224;          // 7 warps: W producer, MMA, 4 epilogue, x producer
#define kPrefetch p.prefetch          // weight tiles requested from HBM into L2 ahead of the ring
constexpr int kEpiThreads = 128;
constexpr int kHeaderBytes = 256;  // status word + padding at the start of the scratch buffer
constexpr int kMaxGrid = 256;      // tickets / partial slots are sized for at most this many CTAs
constexpr int kStageUMax = 8 * 1024;  // shrink outputs are staged in shared memory up to this size

struct TcParams {
  LinearArgs a;
  int k_blocks;    // ceil(in / BK)
  int row_tiles;   // ceil(out / BM)
  int n_tiles;     // row_tiles * token tiles
  int tok_tiles;
  int wave_gt;     // 0: stream-K ranges; > 0: whole tiles, token tiles taken in groups of this many
  int wave_full, wave_ch, wave_ch_last;  // full groups, tiles per CTA in a full group / in the narrower last one
  int wave_lanes;  // > 0: lane form -- CTA c serves token tile (c mod wave_gt) of every group and the row tiles
                   // (c / wave_gt) + s * wave_lanes, s = 0 .. wave_ch - 1; wave_full = number of groups
  int per_cta;     // iterations (tile, k-block) per CTA
  int lora_mode;   // 0 none, 1 expand on CUDA cores in the epilogue, 2 expand on the tensor cores
  int lora_sub;    // K elements of one LoRA stage (16, 32 or 64 = row bytes 32, 64, 128)
  int n_sub;       // LoRA stages per adapter segment (r_max / lora_sub)
  int prefetch;    // weight tiles requested into L2 ahead of the ring (0 = off)
  int tma_store;   // 1: output tiles leave through shared memory + one TMA store per 32-token chunk
  int32_t* status;  // scratch[0]
  int32_t* tickets; // [kMaxGrid], indexed by the first contributing CTA of a split tile
  float* partials;  // [grid][2][BN][BM]
};

// Distinct adapter slots among the tokens of one token tile, in order of first appearance.
// Executed by one full warp; s_tok [BN] receives the tile's slots, s_list [BN] the distinct ones.
template <int BN>
__device__ __forceinline__ int distinct_slots(const LinearArgs& a, int t0, int* s_tok, int* s_list) {
  const int lane = threadIdx.x & 31;
  for (int n = lane; n < BN; n += 32) {
    int s = (t0 + n < a.T) ? a.slots[t0 + n] : -1;
    s_tok[n] = (s >= 0 && s < a.n_adapters) ? s : -1;
  }
  __syncwarp();
  int count = 0;
#pragma unroll 1
  for (int base = 0; base < BN; base += 32) {
    const int n = base + lane;
    const int s = n < BN ? s_tok[n] : -1;
    bool first = s >= 0;
    for (int m = 0; first && m < n; ++m) first = s_tok[m] != s;
    const unsigned mask = __ballot_sync(0xffffffffu, first);
    if (first) s_list[count + __popc(mask & ((1u << lane) - 1))] = s;
    count += __popc(mask);
  }
  __syncwarp();
  return count;
}


// Four adjacent outputs of one token: one 8-byte (bf16) or 16-byte (fp32) store when aligned and
// all four exist, scalar stores otherwise.
__device__ __forceinline__ void store4(const LinearArgs& a, int t, int col, const float (&o)[4], bool out_f32,
                                       int n_valid) {
  const size_t idx = (size_t)t * a.ldy + col;
  if (n_valid >= 4 && (idx & 3) == 0) {
    if (out_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + idx) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
      uint2 v;
      *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(o[0], o[1]);
      *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(o[2], o[3]);
      *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(a.y) + idx) = v;
    }
  } else {
    for (int e = 0; e < 4 && e < n_valid; ++e) {
      if (out_f32)
        reinterpret_cast<float*>(a.y)[idx + e] = o[e];
      else
        reinterpret_cast<bf16*>(a.y)[idx + e] = __float2bfloat16_rn(o[e]);
    }
  }
}

// LoRA expand on CUDA cores for one 32-token chunk of one output row (used only when the tensor-core
// expand does not apply: module boundaries inside a tile).  v[i] += scale * <u[token i], B[slot, row, :]>.
template <int BN>
__device__ __forceinline__ void simt_lora_expand(const LinearArgs& a, float (&v)[32], int c0, int t0, int row,
                                                 int r_tot, bool stage_u, const int* s_slots, const float* s_u) {
  constexpr int kChunk = BN < 32 ? BN : 32;
  if (row >= a.out) return;
  const int m = module_of(a, row);
  int cur = -1, r = 0;
  float sc = 0.f;
  uint4 bq[8];
#pragma unroll
  for (int i = 0; i < kChunk; ++i) {
    const int s = s_slots[c0 + i];
    if (s < 0 || s >= a.n_adapters) continue;
    if (s != cur) {  // rows of one adapter are usually adjacent (ordered batches): reuse B[s, row, :]
      cur = s;
      r = a.full_rank ? a.r_max : a.ranks[s];
      sc = a.scales[s];
      const bf16* b = a.B_all + ((size_t)s * a.out + row) * a.r_max;
#pragma unroll
      for (int g = 0; g < 8; ++g)
        if (g * 8 < r) bq[g] = ld_cached(b + g * 8);
    }
    const float* ur = stage_u ? s_u + (c0 + i) * r_tot + m * a.r_max
                              : a.u + (size_t)(t0 + c0 + i) * r_tot + m * a.r_max;
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (g * 8 < r) {
        float bf[8];
        unpack8(bq[g], bf);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (g * 8 + e < r) acc = fmaf(ur[g * 8 + e], bf[e], acc);
      }
    }
    v[i] = fmaf(sc, acc, v[i]);
  }
}

template <int BN>
struct Cfg {
  static constexpr int kWBytes = BM * BK * 2;    // weight stage: 16 KB
  static constexpr int kXBytes = BN * BK * 2;    // token-tile stage
  // token tiles come from L2: a shallower ring is enough (256-token tiles: three 48 KB stage pairs = 1500 tensor cycles ahead)
  static constexpr int kXStages = BN >= 256 ? 3 : BN >= 64 ? 4 : 8;
  // barriers | 7 integer lists of BN (token slots / distinct adapters per role) | staged shrink outputs
  // LoRA B operands (scaled, masked shrink outputs) of a token tile; prefill-size tiles get room for a rank-128
  // pitch (interleaved gate/up at rank 64) so the operands are built once per token tile, not once per tile
  static constexpr int kCacheBytes = (BN >= 128 ? 64 : 16) * 1024;  // 128-token tiles: 16 rank-16 adapters or 2 of pitch 128
  // shrink outputs of a token tile staged in shared memory (decode-size tiles only; larger tiles read them from L2)
  static constexpr int kStageU = BN >= 128 ? 0 : kStageUMax;
  // staging of one 32-token output chunk; fp32 outputs of 128-token tiles leave through per-thread stores instead
  static constexpr int kOutBytes = 32 * BM * (BN >= 128 ? 2 : 4);
  static constexpr int kAuxBytes = 1024 + 8 * BN * 4 + kStageU + kCacheBytes + kOutBytes + 256 /*s_rstd*/;
  static constexpr int kBudget = 227 * 1024 - 1024 /*alignment slack*/ - 64 /*static*/;
  static constexpr int kWStages0 = (kBudget - kAuxBytes - kXStages * kXBytes) / kWBytes;
  static constexpr int kWStages = kWStages0 > 10 ? 10 : kWStages0;  // measured: 5 stages already saturate
  static constexpr int kSmemBytes = kWStages * kWBytes + kXStages * kXBytes + kAuxBytes + 1024;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // two accumulators
  static constexpr int kChunk = BN < 32 ? BN : 32;              // columns per TMEM load
  static_assert(kWStages >= 3, "weight ring too shallow");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

// Do the LoRA B operands of a token tile with n_seg distinct adapters fit the shared-memory cache?
template <int BN>
__device__ __forceinline__ bool lora_cached(const TcParams& p, int n_seg) {
  return n_seg * p.n_sub * BN * p.lora_sub * 2 <= Cfg<BN>::kCacheBytes;
}

// Prompt-size tiles: are the rows of every adapter of the tile one contiguous run (prompt rows of a request are)?  Then an
// adapter's LoRA stage only needs the 16-row blocks its rows touch: its B operand has `rows` = the run rounded out to 16
// rows, and its MMAs write the accumulator columns [first, first + rows) with N = rows.  All operands of a tile then take
// BN + 16 rows per adapter at most, whatever the number of adapters.  Returns the total number of operand rows, or -1 when
// some adapter's rows are scattered (or there are more than 16 adapters).  One full warp; s_tok / s_list as written by
// distinct_slots; tab (optional, [16]): per adapter (first accumulator column, rows, row offset of its operand).
template <int BN>
__device__ __forceinline__ int adapter_runs(const int* s_tok, const int* s_list, int n_seg, int4* tab) {
  if (BN < 128 || n_seg > 16) return -1;
  const int lane = threadIdx.x & 31;
  int total = 0;
  bool ok = true;
  for (int j = 0; j < n_seg; ++j) {
    const int s = s_list[j];
    int lo = BN, hi = -1, cnt = 0;
    for (int r = lane; r < BN; r += 32)
      if (s_tok[r] == s) {
        lo = min(lo, r);
        hi = max(hi, r);
        ++cnt;
      }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    cnt = __reduce_add_sync(0xffffffffu, cnt);
    ok = ok && cnt == hi - lo + 1;
    const int first = lo & ~15, rows = ((hi + 16) & ~15) - first;
    if (tab != nullptr && lane == 0) tab[j] = make_int4(first, rows, total, 0);
    total += rows;
  }
  return ok ? total : -1;
}
// Operands of a tile in the shared-memory cache: in the run layout when the rows allow it and it fits, else as full-height
// masked operands per adapter when those fit.
template <int BN>
__device__ __forceinline__ bool lora_runs(const TcParams& p, int n_run) {
  return BN >= 128 && n_run >= 0 && n_run * p.n_sub * p.lora_sub * 2 <= Cfg<BN>::kCacheBytes;
}
template <int BN>
__device__ __forceinline__ bool lora_in_cache(const TcParams& p, int n_seg, int n_run) {
  return lora_runs<BN>(p, n_run) || lora_cached<BN>(p, n_seg);
}

// One CTA's share of the iteration space and the walk over its segments.
struct Range {
  int it0, it1;
};
struct Segment {
  int tile, kb0, kb1;
};
// Prefill sizes (many token tiles): whole tiles only.  The token tiles are taken in groups of `wave_gt`, so that at
// any time the grid works on wave_gt token tiles (L2 resident) and a handful of row tiles that many CTAs share,
// instead of every CTA pulling its own operands from HBM; and a CTA's consecutive tiles share the token tile (and
// mostly the module), so the LoRA operands it caches in shared memory are rebuilt rarely.  Two ways of dealing a
// group's tiles: the lane form (default, below), and the chunk form -- tiles ordered token tile major / row tile
// minor and cut into equal contiguous chunks, one per CTA, which only keeps the CTAs on shared row tiles when the
// chunk length divides the row tiles.
// Slot `lt` of this CTA's walk -> tile id (token tile * row_tiles + row tile), or -1 where its chunk of that
// group is shorter than the longest.
__device__ __forceinline__ int wave_tile(const TcParams& p, int lt) {
  if (p.wave_lanes > 0) {
    // lane form: at step s the CTAs of one lane -- one per token tile of the group -- all read row tile lane + s * lanes,
    // so a weight tile comes from HBM once per group and from L2 for the other wave_gt - 1 CTAs
    const int grp = lt / p.wave_ch, st = lt - grp * p.wave_ch;
    const int j = (int)blockIdx.x % p.wave_gt, lane = (int)blockIdx.x / p.wave_gt;
    const int row = lane + st * p.wave_lanes, tok = grp * p.wave_gt + j;
    if (lane >= p.wave_lanes || row >= p.row_tiles || tok >= p.tok_tiles) return -1;
    return tok * p.row_tiles + row;
  }
  int group, qi, gt, ch;
  const int full_slots = p.wave_full * p.wave_ch;
  if (lt < full_slots) {
    group = lt / p.wave_ch;
    qi = lt - group * p.wave_ch;
    gt = p.wave_gt;
    ch = p.wave_ch;
  } else {
    group = p.wave_full;
    qi = lt - full_slots;
    gt = p.tok_tiles - group * p.wave_gt;
    ch = p.wave_ch_last;
  }
  const int q = (int)blockIdx.x * ch + qi;
  if (q >= p.row_tiles * gt) return -1;
  const int j = q / p.row_tiles;
  return (group * p.wave_gt + j) * p.row_tiles + (q - j * p.row_tiles);
}
template <bool WAVE>
__device__ __forceinline__ Range cta_range(const TcParams& p, int cta) {
  if (WAVE && p.wave_gt > 0) return Range{0, (p.wave_full * p.wave_ch + p.wave_ch_last) * p.k_blocks};
  const long long total = (long long)p.n_tiles * p.k_blocks;
  long long a = (long long)cta * p.per_cta, b = a + p.per_cta;
  if (a > total) a = total;
  if (b > total) b = total;
  return Range{(int)a, (int)b};
}
// Next piece of work of this CTA; tile < 0: none left.  WAVE = false compiles the whole-tile walk out (the
// decode-size instantiations are sensitive to code size).
template <bool WAVE>
__device__ __forceinline__ Segment next_segment(const TcParams& p, int& it, int it1) {
  Segment s;
  if (WAVE && p.wave_gt > 0) {
    s.tile = -1;
    s.kb0 = 0;
    s.kb1 = p.k_blocks;
    while (it < it1 && s.tile < 0) {
      s.tile = wave_tile(p, it / p.k_blocks);
      it += p.k_blocks;
    }
    return s;
  }
  s.tile = it / p.k_blocks;
  s.kb0 = it - s.tile * p.k_blocks;
  s.kb1 = min(p.k_blocks, s.kb0 + (it1 - it));
  it += s.kb1 - s.kb0;
  return s;
}

// LM: 0 = no LoRA code at all, 1 = expand on CUDA cores in the epilogue, 2 = expand as extra MMA stages when
// p.lora_mode == 2 (this instantiation also serves base-only calls flagged MLORA_SHARE_LORA_KERNEL).  Separate
// instantiations because the decode-size kernels are sensitive to code size: every launch starts with cold
// instruction caches after 100+ MB of weights went through L2, so a step whose projections alternate between two
// instantiations pays for two code footprints; one that uses a single instantiation throughout does not.
// NF: the folded residual + RMSNorm epilogues (NormFuse) are compiled in.  Its own instantiation: the extra code and
// registers (233 against 164 per thread at 32-token tiles) cost every launch of the kernel ~0.3 us even when unused.
template <int BN, int LM, bool NF = false>
__global__ void __launch_bounds__(kThreads, 1) linear_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                const __grid_constant__ CUtensorMap map_b,
                                                                const __grid_constant__ CUtensorMap map_y,
                                                                TcParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* w_ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* x_ring = w_ring + C::kWStages * C::kWBytes;
  uint8_t* s_cache = x_ring + C::kXStages * C::kXBytes;  // 1024-byte aligned like the rings
  uint8_t* s_out = s_cache + C::kCacheBytes;             // output staging for the TMA store
  uint8_t* aux = s_out + C::kOutBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(aux);  // [kWStages] weight stage filled
  uint64_t* empty_bar = full_bar + C::kWStages;           // [kWStages] weight stage consumed
  uint64_t* xfull_bar = empty_bar + C::kWStages;          // [kXStages]
  uint64_t* xempty_bar = xfull_bar + C::kXStages;         // [kXStages]
  uint64_t* acc_full = xempty_bar + C::kXStages;          // [2]
  uint64_t* acc_empty = acc_full + 2;                     // [2]
  uint64_t* cache_full = acc_empty + 2;                   // LoRA operand cache written / all readers retired
  uint64_t* cache_empty = cache_full + 1;
  uint64_t* preload_bar = cache_empty + 1;                // LoRA operands of the first token tile are in smem
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(preload_bar + 1);
  int* s_slots = reinterpret_cast<int*>(aux + 1024);  // [BN] epilogue warps (CUDA-core expand)
  int* p_tok = s_slots + BN;                           // weight producer: slots of the token tile
  int* p_list = p_tok + BN;                            //                  distinct slots
  int* m_tok = p_list + BN;                            // MMA warp
  int* m_list = m_tok + BN;
  int* x_tok = m_list + BN;                            // token-tile producer
  int* x_list = x_tok + BN;
  float* x_scale = reinterpret_cast<float*>(x_list + BN);  // scale of each distinct slot
  float* s_u = x_scale + BN;                           // [BN * r_tot] when it fits
  float* s_red = reinterpret_cast<float*>(aux + 512);                   // [4][32] per-warp partial sums of squares (NormFuse)
  // prompt-size tiles: the output warps build the cached LoRA operands (their own list of the tile's adapters; the
  // cache holds at most 16 of them)
  int* e_list = reinterpret_cast<int*>(aux + 512);                      // [16]  (decode-size tiles use this space as s_red)
  float* e_scale = reinterpret_cast<float*>(aux + 512 + 64);            // [16]
  int4* e_tab = reinterpret_cast<int4*>(aux + 512 + 128);               // [16] run layout: (first column, rows, operand row offset)
  int* e_nrun = reinterpret_cast<int*>(aux + 512 + 128 + 256);
  // (kAuxBytes also counts the operand cache and the output staging, which lie BEFORE aux: address from aux's own parts)
  float* s_rstd = reinterpret_cast<float*>(aux + 1024 + 8 * BN * 4 + C::kStageU);  // [32] 1/rms of the input rows (NormFuse consumer)
  __shared__ int s_abort;
  __shared__ int s_last;
  __shared__ int s_nseg0;  // distinct adapters of the CTA's first token tile (listed before the roles start)
  __shared__ int s_runs0;  // ... and their operand rows in the run layout (adapter_runs)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool WAVE = BN >= 128;  // prefill-size token tiles only
  const Range rg = cta_range<WAVE>(p, blockIdx.x);
  if (rg.it0 >= rg.it1) return;  // whole CTA idle (uniform)
  const LinearArgs& a = p.a;
  const int r_tot = a.r_max * a.n_mod;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < C::kWStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < C::kXStages; ++s) {
      mbar_init(&xfull_bar[s], 1);
      mbar_init(&xempty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
    }
    mbar_init(cache_full, 1);
    mbar_init(cache_empty, 1);
    mbar_init(preload_bar, 4);  // the four epilogue warps
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!(a.flags & MLORA_W_PACKED)) tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
    if ((LM == 2 && p.lora_mode == 2) && !(a.flags & MLORA_B_PACKED)) tma_prefetch_desc(&map_b);
    if (p.tma_store) tma_prefetch_desc(&map_y);
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // From here on the next kernel in the stream may become resident; this kernel's weight producer
  // starts streaming at once (weights are constant inputs), every other role first waits until the
  // kernels before it have completed.
  pdl_launch_dependents();
  int first_it = rg.it0;
  const int first_tile = next_segment<WAVE>(p, first_it, rg.it1).tile;
  const int tok_tile0 = (first_tile < 0 ? 0 : first_tile) / p.row_tiles;
  const bool stage_u2 = (LM == 2 && p.lora_mode == 2) && (size_t)BN * r_tot * sizeof(float) <= (size_t)C::kStageU;
  if (warp != 0) pdl_wait();
  if ((LM == 2 && p.lora_mode == 2) && warp >= 2 && warp <= 5) {
    // The per-token LoRA operands of the CTA's first token tile (decode: the only one) are fetched now,
    // by the epilogue warps, which are idle at start-up, so that no pipeline role stops mid-stream for a
    // global load.  The roles pick the result up through `preload_bar` when they first need it.
    if (warp == 2) {
      const int ns = distinct_slots<BN>(a, tok_tile0 * BN, p_tok, p_list);
      const int nr = adapter_runs<BN>(p_tok, p_list, ns, nullptr);
      if (lane == 0) s_runs0 = nr;
      for (int i = lane; i < BN; i += 32) {
        m_tok[i] = x_tok[i] = p_tok[i];
        if (i < ns) {
          m_list[i] = x_list[i] = p_list[i];
          x_scale[i] = a.scales[p_list[i]];
        }
      }
      if (lane == 0) s_nseg0 = ns;
    } else if (stage_u2) {
      // all loads of a thread are issued before the first store (r_tot is a multiple of 8: float4 granules)
      const int n_vec = min(BN, a.T - tok_tile0 * BN) * r_tot / 4;
      const float4* src = reinterpret_cast<const float4*>(a.u + (size_t)tok_tile0 * BN * r_tot);
      float4 tmp[8];
      for (int base = (warp - 3) * 32 + lane; base < n_vec; base += 96 * 8) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (base + c * 96 < n_vec) tmp[c] = __ldg(src + base + c * 96);
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (base + c * 96 < n_vec) reinterpret_cast<float4*>(s_u)[base + c * 96] = tmp[c];
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(preload_bar);
  }
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t rb = p.lora_sub * 2;  // row bytes of a LoRA stage

  if (warp == 0) {
    // ---- weight producer: lane 0 issues the copies; all lanes list the adapters of a token tile ------
    const bool packed = (a.flags & MLORA_W_PACKED) != 0;
    const uint8_t* wp = reinterpret_cast<const uint8_t*>(a.W);
    int it = rg.it0, n = 0, cur_tok_tile = tok_tile0, n_seg = 0, n_run = -1;
    bool got_preload = false;
    bool ok = true;
    // decode sizes read every weight byte once: "evict first", so that the stream does not push token tiles, partial
    // sums and the kernel's instructions out of L2; prefill sizes re-read weight tiles from L2 and keep the default
    const bool stream_once = !WAVE || p.wave_gt == 0;
    const uint64_t pol = l2_policy_evict_first();
    while (it < rg.it1 && ok) {
      const Segment sg = next_segment<WAVE>(p, it, rg.it1);
      if (WAVE && sg.tile < 0) break;
      const int row_tile = sg.tile % p.row_tiles, tok_tile = sg.tile / p.row_tiles;
      if (lane == 0) {
        int nn = n;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++nn) {
          const int s = nn % C::kWStages, round = nn / C::kWStages;
          if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &s_abort)) {
            s_abort = 1;
            atomicOr(p.status, 1);
            ok = false;
            break;
          }
          uint8_t* st = w_ring + s * C::kWBytes;
          mbar_expect_tx(&full_bar[s], C::kWBytes);
          if (packed && stream_once)  // one contiguous 16 KB tile, already in the swizzled K-major layout
            bulk_load_hint(st, wp + ((size_t)row_tile * p.k_blocks + kb) * C::kWBytes, C::kWBytes, &full_bar[s], pol);
          else if (packed)
            bulk_load(st, wp + ((size_t)row_tile * p.k_blocks + kb) * C::kWBytes, C::kWBytes, &full_bar[s]);
          else
            tma_load_2d(st, &map_w, kb * BK, row_tile * BM, &full_bar[s]);
        }
      }
      n += sg.kb1 - sg.kb0;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok && (LM == 2 && p.lora_mode == 2) && sg.kb0 == 0) {
        if (!got_preload) {  // operands of the first token tile, staged by the epilogue warps at start-up
          mbar_wait(preload_bar, 0, &s_abort);
          n_seg = s_nseg0;
          n_run = s_runs0;
          got_preload = true;
        }
        // The tile's first k-blocks are ours: this CTA also runs the tile's LoRA stages, after them.  (For a split
        // tile that is the CTA that finishes it, at the END of its range, when the shrink outputs have long been
        // staged and the operands built; the CTA holding the tile's last k-blocks reaches them at the very start
        // of its range and would have to wait for all that first.)  One stage per (adapter present in
        // the token tile, 64-wide slice of the rank); its A operand is B_all[slot, rows of the tile, slice].
        // When the B operands are cached in shared memory, up to `group` such slices share one ring slot.
        if (tok_tile != cur_tok_tile) {
          n_seg = distinct_slots<BN>(a, tok_tile * BN, p_tok, p_list);
          n_run = adapter_runs<BN>(p_tok, p_list, n_seg, nullptr);
          cur_tok_tile = tok_tile;
        }
        const int n_l = n_seg * p.n_sub;
        const int group = lora_in_cache<BN>(p, n_seg, n_run) ? C::kWBytes / (BM * (int)rb) : 1;
        const int n_groups = (n_l + group - 1) / group;
        if (lane == 0) {
          int nn = n;
          for (int g = 0; g < n_groups && ok; ++g, ++nn) {
            const int s = nn % C::kWStages, round = nn / C::kWStages;
            if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &s_abort)) {
              s_abort = 1;
              atomicOr(p.status, 1);
              ok = false;
              break;
            }
            const int l0 = g * group, l1 = min(n_l, l0 + group);
            mbar_expect_tx(&full_bar[s], (l1 - l0) * BM * rb);
            for (int l = l0; l < l1; ++l) {
              const int slot = p_list[l / p.n_sub], sb = l % p.n_sub;
              uint8_t* dst = w_ring + s * C::kWBytes + (l - l0) * BM * rb;
              if (a.flags & MLORA_B_PACKED)  // one contiguous pre-swizzled tile
                bulk_load(dst, reinterpret_cast<const uint8_t*>(a.B_all) +
                                   (((size_t)slot * p.row_tiles + row_tile) * p.n_sub + sb) * (BM * rb),
                          BM * rb, &full_bar[s]);
              else
                tma_load_2d(dst, &map_b, sb * p.lora_sub, slot * a.out + row_tile * BM, &full_bar[s]);
            }
          }
        }
        n += n_groups;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
  } else if (warp == 6) {
    // ---- token-tile producer: lane 0 issues the x copies; all lanes build the LoRA B operands --------
    const bool stage_u = stage_u2;
    int it = rg.it0, n = 0, cur_tok_tile = tok_tile0, n_seg = 0, n_run = -1, cur_key = -1, n_build = 0;
    bool got_preload = false;
    bool ok = true;
    while (it < rg.it1 && ok) {
      const Segment sg = next_segment<WAVE>(p, it, rg.it1);
      if (WAVE && sg.tile < 0) break;
      const int row_tile = sg.tile % p.row_tiles, tok_tile = sg.tile / p.row_tiles;
      if (lane == 0) {
        int nn = n;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++nn) {
          const int s = nn % C::kXStages, round = nn / C::kXStages;
          if (!mbar_wait(&xempty_bar[s], (round & 1) ^ 1, &s_abort)) {
            s_abort = 1;
            atomicOr(p.status, 16);
            ok = false;
            break;
          }
          mbar_expect_tx(&xfull_bar[s], C::kXBytes);
          tma_load_2d(x_ring + s * C::kXBytes, &map_x, kb * BK, tok_tile * BN, &xfull_bar[s]);
        }
      }
      n += sg.kb1 - sg.kb0;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (ok && (LM == 2 && p.lora_mode == 2) && sg.kb0 == 0) {
        if (!got_preload) {  // operands of the first token tile, staged by the epilogue warps at start-up
          mbar_wait(preload_bar, 0, &s_abort);
          n_seg = s_nseg0;
          n_run = s_runs0;
          got_preload = true;
        }
        // B operand of a LoRA stage = scale * u of the tokens that use the adapter (zero rows for the
        // others), written in the swizzled K-major layout the MMA expects: once per (token tile, module)
        // into the shared-memory cache when all of them fit, else stage by stage into the x ring.
        const int t0 = tok_tile * BN;
        if (tok_tile != cur_tok_tile) {
          n_seg = distinct_slots<BN>(a, t0, x_tok, x_list);
          n_run = adapter_runs<BN>(x_tok, x_list, n_seg, nullptr);
          for (int i = lane; i < n_seg; i += 32) x_scale[i] = a.scales[x_list[i]];
          if (stage_u) {
            const int n_valid = min(BN, a.T - t0) * r_tot;
            for (int i = lane; i < n_valid; i += 32) s_u[i] = a.u[(size_t)t0 * r_tot + i];
            __syncwarp();
          }
          cur_tok_tile = tok_tile;
        }
        const int mod = module_of(a, row_tile * BM);
        const int u_off = mod * a.r_max;
        const int chunks = p.lora_sub / 8;  // 16-byte chunks per row
        const bool cached = lora_in_cache<BN>(p, n_seg, n_run);
        if (BN >= 128 && cached) continue;  // prompt-size tiles: the output warps build the cache (below)
        if (cached && tok_tile * 8 + mod == cur_key) continue;  // operands already in the cache
        if (cached) {
          int w = 1;
          if (lane == 0) w = mbar_wait(cache_empty, (n_build & 1) ^ 1, &s_abort) ? 1 : 0;
          w = __shfl_sync(0xffffffffu, w, 0);
          if (!w) {
            if (lane == 0) {
              s_abort = 1;
              atomicOr(p.status, 32);
            }
            break;
          }
        }
        if (cached) {
          // zero the tiles, then drop each token's scaled shrink output into the tile of its adapter
          const int n_vec = n_seg * p.n_sub * BN * (int)rb / 16;
          for (int i = lane; i < n_vec; i += 32) reinterpret_cast<uint4*>(s_cache)[i] = make_uint4(0u, 0u, 0u, 0u);
          __syncwarp();
          const int per_row = chunks * p.n_sub;
          if constexpr (BN >= 128) {
            // four items per lane and step, their shrink outputs requested before the first is used (the
            // loads are L2 round trips when the outputs are not staged in shared memory)
            for (int base = lane; base < BN * per_row; base += 32 * 4) {
              float4 lo[4], hi[4];
              int nr[4], off[4];
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const int idx = base + b * 32;
                nr[b] = -1;
                if (idx < BN * per_row) {
                  const int nrow = idx / per_row, rem = idx - nrow * per_row;
                  const int sb = rem / chunks, c = rem - sb * chunks;
                  if (x_tok[nrow] >= 0) {
                    nr[b] = nrow;
                    off[b] = sb * 256 + c;
                    const float* ur = (stage_u ? s_u + nrow * r_tot : a.u + (size_t)(t0 + nrow) * r_tot) + u_off +
                                      sb * p.lora_sub + c * 8;
                    lo[b] = *reinterpret_cast<const float4*>(ur);
                    hi[b] = *reinterpret_cast<const float4*>(ur + 4);
                  }
                }
              }
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                if (nr[b] < 0) continue;
                const int nrow = nr[b], sb = off[b] >> 8, c = off[b] & 255;
                const int slot = x_tok[nrow];
                int sgi = 0;
                while (x_list[sgi] != slot) ++sgi;  // slot is in the list by construction
                const float sc = x_scale[sgi];
                const float f[8] = {lo[b].x * sc, lo[b].y * sc, lo[b].z * sc, lo[b].w * sc,
                                    hi[b].x * sc, hi[b].y * sc, hi[b].z * sc, hi[b].w * sc};
                const int sw = rb == 128 ? (nrow & 7) : rb == 64 ? ((nrow >> 1) & 3) : ((nrow >> 2) & 1);
                *reinterpret_cast<uint4*>(s_cache + (sgi * p.n_sub + sb) * BN * rb + nrow * rb + ((c ^ sw) << 4)) = pack8(f);
              }
            }
          } else {
            for (int idx = lane; idx < BN * per_row; idx += 32) {
              const int nrow = idx / per_row, rem = idx - nrow * per_row;
              const int sb = rem / chunks, c = rem - sb * chunks;
              const int slot = x_tok[nrow];
              if (slot < 0) continue;
              int sgi = 0;
              while (x_list[sgi] != slot) ++sgi;  // slot is in the list by construction
              const float sc = x_scale[sgi];
              const float* ur = (stage_u ? s_u + nrow * r_tot : a.u + (size_t)(t0 + nrow) * r_tot) + u_off +
                                sb * p.lora_sub + c * 8;
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = ur[e] * sc;
              const int sw = rb == 128 ? (nrow & 7) : rb == 64 ? ((nrow >> 1) & 3) : ((nrow >> 2) & 1);
              *reinterpret_cast<uint4*>(s_cache + (sgi * p.n_sub + sb) * BN * rb + nrow * rb + ((c ^ sw) << 4)) = pack8(f);
            }
          }
        }
        for (int sgi = 0; sgi < n_seg && ok && !cached; ++sgi) {
          const int slot = x_list[sgi];
          const float sc = x_scale[sgi];
          for (int sb = 0; sb < p.n_sub; ++sb) {
            const int s = n % C::kXStages, round = n / C::kXStages;
            int w = 1;
            if (lane == 0) w = mbar_wait(&xempty_bar[s], (round & 1) ^ 1, &s_abort) ? 1 : 0;
            w = __shfl_sync(0xffffffffu, w, 0);
            if (!w) {
              if (lane == 0) {
                s_abort = 1;
                atomicOr(p.status, 16);
              }
              ok = false;
              break;
            }
            uint8_t* xt = x_ring + s * C::kXBytes;
            if constexpr (BN >= 128) {
              // four items per lane and step, their shrink outputs (L2 round trips) requested before the first is used
              for (int base = lane; base < BN * chunks; base += 32 * 4) {
                float4 lo[4], hi[4];
                bool mine[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  const int idx = base + b * 32;
                  const int nrow = idx / chunks, c = idx - nrow * chunks;
                  mine[b] = idx < BN * chunks && x_tok[nrow] == slot;
                  if (mine[b]) {
                    const float* ur = a.u + (size_t)(t0 + nrow) * r_tot + u_off + sb * p.lora_sub + c * 8;
                    lo[b] = *reinterpret_cast<const float4*>(ur);
                    hi[b] = *reinterpret_cast<const float4*>(ur + 4);
                  }
                }
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  const int idx = base + b * 32;
                  if (idx >= BN * chunks) continue;
                  const int nrow = idx / chunks, c = idx - nrow * chunks;
                  uint4 val = make_uint4(0u, 0u, 0u, 0u);
                  if (mine[b]) {
                    const float f[8] = {lo[b].x * sc, lo[b].y * sc, lo[b].z * sc, lo[b].w * sc,
                                        hi[b].x * sc, hi[b].y * sc, hi[b].z * sc, hi[b].w * sc};
                    val = pack8(f);
                  }
                  const int sw = rb == 128 ? (nrow & 7) : rb == 64 ? ((nrow >> 1) & 3) : ((nrow >> 2) & 1);
                  *reinterpret_cast<uint4*>(xt + nrow * rb + ((c ^ sw) << 4)) = val;
                }
              }
            } else {
              for (int idx = lane; idx < BN * chunks; idx += 32) {
                const int nrow = idx / chunks, c = idx - nrow * chunks;
                uint4 val = make_uint4(0u, 0u, 0u, 0u);
                if (x_tok[nrow] == slot) {
                  const float* ur = (stage_u ? s_u + nrow * r_tot : a.u + (size_t)(t0 + nrow) * r_tot) + u_off +
                                    sb * p.lora_sub + c * 8;
                  float f[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) f[e] = ur[e] * sc;
                  val = pack8(f);
                }
                const int sw = rb == 128 ? (nrow & 7) : rb == 64 ? ((nrow >> 1) & 3) : ((nrow >> 2) & 1);
                *reinterpret_cast<uint4*>(xt + nrow * rb + ((c ^ sw) << 4)) = val;
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&xfull_bar[s]);
            ++n;
          }
        }
        if (cached && ok) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(cache_full);
          cur_key = tok_tile * 8 + mod;
          ++n_build;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: lane 0 issues; all lanes count the LoRA stages of a token tile ---------------------
    constexpr uint32_t idesc = make_idesc(BM, BN);
    int it = rg.it0, nw = 0, nx = 0, j = 0, cur_tok_tile = tok_tile0, n_seg = 0, n_run = -1, cur_key = -1, n_build = 0;
    bool got_preload = false;
    bool ok = true;
    while (it < rg.it1 && ok) {
      const Segment sg = next_segment<WAVE>(p, it, rg.it1);
      if (WAVE && sg.tile < 0) break;
      const int row_tile = sg.tile % p.row_tiles, tok_tile = sg.tile / p.row_tiles;
      const int buf = j & 1;
      const uint32_t d_tmem = tmem_base + buf * BN;
      int n_l = 0, group = 1;
      bool cached = false, new_build = false;
      if ((LM == 2 && p.lora_mode == 2) && sg.kb0 == 0) {
        if (!got_preload) {  // operands of the first token tile, staged by the epilogue warps at start-up
          mbar_wait(preload_bar, 0, &s_abort);
          n_seg = s_nseg0;
          n_run = s_runs0;
          got_preload = true;
        }
        if (tok_tile != cur_tok_tile) {
          n_seg = distinct_slots<BN>(a, tok_tile * BN, m_tok, m_list);
          n_run = adapter_runs<BN>(m_tok, m_list, n_seg, nullptr);
          cur_tok_tile = tok_tile;
        }
        n_l = n_seg * p.n_sub;
        cached = lora_in_cache<BN>(p, n_seg, n_run);
        if (cached) {
          group = C::kWBytes / (BM * (int)rb);
          const int key = tok_tile * 8 + module_of(a, row_tile * BM);
          new_build = key != cur_key;
          cur_key = key;
        }
      }
      const int n_groups = (n_l + group - 1) / group;
      const int n_w = sg.kb1 - sg.kb0;
      if (lane == 0) {
        int w_i = nw, x_i = nx;
        if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, &s_abort)) {
          s_abort = 1;
          atomicOr(p.status, 8);
          ok = false;
        }
        tc_fence_after();
        {
          // The stream's inner loop, one thread: ring positions, parities, barrier addresses and descriptors are
          // kept in registers and advanced by additions (no division, no address conversion per stage).
          int ws = w_i % C::kWStages, xs = x_i % C::kXStages;
          uint32_t wpar = (w_i / C::kWStages) & 1, xpar = (x_i / C::kXStages) & 1;
          const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
          const uint32_t xfull0 = smem_u32(xfull_bar), xempty0 = smem_u32(xempty_bar);
          const uint64_t adesc0 = make_smem_desc(smem_u32(w_ring)), bdesc0 = make_smem_desc(smem_u32(x_ring));
          for (int l = 0; l < n_w && ok; ++l) {
            if (!mbar_wait_a(full0 + 8 * ws, wpar, &s_abort) || !mbar_wait_a(xfull0 + 8 * xs, xpar, &s_abort)) {
              s_abort = 1;
              atomicOr(p.status, 2);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint64_t adesc = adesc0 + (uint64_t)(ws * (C::kWBytes >> 4));  // start-address field, 16-byte units
            const uint64_t bdesc = bdesc0 + (uint64_t)(xs * (C::kXBytes >> 4));
            umma_bf16(d_tmem, adesc, bdesc, idesc, l > 0 ? 1u : 0u);
#pragma unroll
            for (int k = 1; k < BK / 16; ++k)  // +16 elements (32 bytes) along K = +2 in the address field
              umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
            umma_commit_a(empty0 + 8 * ws);  // both stages are free once these MMAs have read them
            umma_commit_a(xempty0 + 8 * xs);
            if (++ws == C::kWStages) {
              ws = 0;
              wpar ^= 1;
            }
            if (++xs == C::kXStages) {
              xs = 0;
              xpar ^= 1;
            }
            ++w_i;
            ++x_i;
          }
        }
        if (cached && new_build && ok) {
          // every MMA that read the previous cache contents has been issued: let the builder overwrite
          // them once those MMAs retire, then wait for the new contents
          if (BN < 128 && n_build > 0) umma_commit(cache_empty);  // (prompt sizes: the builders order themselves by acc_full)
          if (!mbar_wait(cache_full, n_build & 1, &s_abort)) {
            s_abort = 1;
            atomicOr(p.status, 64);
            ok = false;
          }
          tc_fence_after();
        }
        for (int g = 0; g < n_groups && ok; ++g, ++w_i) {
          const int s = w_i % C::kWStages;
          int xs = 0;
          bool got = mbar_wait(&full_bar[s], (w_i / C::kWStages) & 1, &s_abort);
          if (got && !cached) {
            xs = x_i % C::kXStages;
            got = mbar_wait(&xfull_bar[xs], (x_i / C::kXStages) & 1, &s_abort);
          }
          if (!got) {
            s_abort = 1;
            atomicOr(p.status, 2);
            ok = false;
            break;
          }
          tc_fence_after();
          const int l0 = g * group, l1 = min(n_l, l0 + group);
          for (int l = l0; l < l1; ++l) {
            const uint64_t adesc = make_smem_desc(smem_u32(w_ring + s * C::kWBytes + (l - l0) * BM * rb), rb);
            if (cached && lora_runs<BN>(p, n_run)) {
              // run layout (written, with its table, by the output warps): only the adapter's own 16-row blocks
              const int sgi = l / p.n_sub, sb = l - sgi * p.n_sub;
              const int4 tb = e_tab[sgi];
              const uint64_t bdesc = make_smem_desc(smem_u32(s_cache + (size_t)(tb.z * p.n_sub + sb * tb.y) * rb), rb);
              const uint32_t idesc_run = make_idesc(BM, tb.y);
              for (int k = 0; k < p.lora_sub / 16; ++k) umma_bf16(d_tmem + tb.x, adesc + 2 * k, bdesc + 2 * k, idesc_run, 1u);
              continue;
            }
            const uint64_t bdesc = make_smem_desc(
                cached ? smem_u32(s_cache + l * BN * rb) : smem_u32(x_ring + xs * C::kXBytes), rb);
            for (int k = 0; k < p.lora_sub / 16; ++k) umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
          }
          umma_commit(&empty_bar[s]);
          if (!cached) {
            umma_commit(&xempty_bar[xs]);
            ++x_i;
          }
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
      nw += n_w + n_groups;
      nx += n_w + (cached ? 0 : n_groups);
      if (cached && new_build) ++n_build;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      ++j;
    }
  } else {
    // ---- epilogue warps 2..5: TMEM lane quarter = warp % 4 ------------------------------------------------
    const int q = warp & 3;
    const int etid = q * 32 + lane;           // 0..127 = row inside the tile
    const bool silu = (a.flags & MLORA_SILU_MUL) != 0;
    const bool out_f32 = (a.flags & MLORA_OUT_F32) != 0;
    constexpr bool simt_lora = LM == 1;
    const bool stage_u = simt_lora && (size_t)BN * r_tot * sizeof(float) <= (size_t)C::kStageU;
    int staged_tok_tile = -1;
    int it = rg.it0, j = 0;
    int e_tok_tile = -1, e_nseg = 0, e_run = -1, e_key = -1;  // prompt-size tiles: the output warps' view of the LoRA operand cache
    const NormFuse& nf = a.nf;
    if constexpr (BN <= 32 && NF) {
      if (nf.sumsq_in != nullptr) {  // (uniform) 1/rms of the input rows from the producer's per-tile sums of squares
        if (etid < 32) {
          float s = 0.f;
#pragma unroll 8
          for (int jj = 0; jj < nf.n_sumsq_in; ++jj) s += __ldcg(nf.sumsq_in + (size_t)jj * 32 + etid);
          s_rstd[etid] = rsqrtf(s / (float)nf.norm_dim + nf.eps);
        }
        epi_bar_sync();
      }
    }

    while (it < rg.it1) {
      const Segment sg = next_segment<WAVE>(p, it, rg.it1);
      if (WAVE && sg.tile < 0) break;
      const int row_tile = sg.tile % p.row_tiles, tok_tile = sg.tile / p.row_tiles;
      const int row = row_tile * BM + etid;
      const int t0 = tok_tile * BN;
      const int buf = j & 1;
      const bool full_seg = sg.kb0 == 0 && sg.kb1 == p.k_blocks;

      // per-token LoRA operands of this token tile -> shared memory (CUDA-core expand only)
      if (simt_lora && staged_tok_tile != tok_tile) {
        epi_bar_sync();  // previous users of the staging area are done
        for (int i = etid; i < BN; i += kEpiThreads) s_slots[i] = (t0 + i < a.T) ? a.slots[t0 + i] : -1;
        if (stage_u) {
          const int n_valid = min(BN, a.T - t0) * r_tot;
          for (int i = etid; i < n_valid; i += kEpiThreads) s_u[i] = a.u[(size_t)t0 * r_tot + i];
        }
        epi_bar_sync();
        staged_tok_tile = tok_tile;
      }

      // Prompt-size tiles: the LoRA B operands of this (token tile, module) -- scale * u of the rows that use the adapter,
      // zero rows for the others, swizzled K-major -- are built HERE, by the 128 threads of the output warps, while the
      // tile's MMAs run: these warps have just finished the previous tile's epilogue, i.e. every MMA that read the old
      // cache contents has retired (its accumulator was complete), and the token-tile producer keeps issuing copies
      // instead of stopping for a chain of L2 round trips at every change of module.
      if constexpr (BN >= 128 && LM == 2) {
        if (p.lora_mode == 2 && sg.kb0 == 0) {  // (the CTA that holds a tile's first k-blocks runs its LoRA stages)
          if (tok_tile != e_tok_tile) {
            // the tile's adapters, listed by one warp; the output staging area serves as its scratch list
            if (etid == 0) bulk_wait_read0();  // the last store has finished reading it
            epi_bar_sync();                    // ... and nobody still reads the previous list
            if (q == 0) {
              int* scratch = reinterpret_cast<int*>(s_out);
              const int ns = distinct_slots<BN>(a, t0, s_slots, scratch);
              const int nr = adapter_runs<BN>(s_slots, scratch, ns, e_tab);
              for (int i = lane; i < ns && i < 16; i += 32) {
                e_list[i] = scratch[i];
                e_scale[i] = a.scales[scratch[i]];
              }
              if (lane == 0) {
                s_last = ns;
                *e_nrun = nr;
              }
            }
            epi_bar_sync();
            e_nseg = s_last;
            e_run = *e_nrun;
            e_tok_tile = tok_tile;
            epi_bar_sync();  // s_last is reused by the split-tile hand-off
          }
          const int mod = module_of(a, row_tile * BM);
          if (lora_in_cache<BN>(p, e_nseg, e_run) && tok_tile * 8 + mod != e_key) {
            const bool runs = lora_runs<BN>(p, e_run);
            const int chunks = p.lora_sub / 8, per_row = chunks * p.n_sub, u_off = mod * a.r_max;
            const int n_vec = (runs ? e_run : e_nseg * BN) * p.n_sub * (int)rb / 16;
            for (int i = etid; i < n_vec; i += kEpiThreads) reinterpret_cast<uint4*>(s_cache)[i] = make_uint4(0u, 0u, 0u, 0u);
            epi_bar_sync();
            for (int base = etid; base < BN * per_row; base += kEpiThreads * 4) {
              float4 lo[4], hi[4];
              int nr[4], off[4];
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const int idx = base + b * kEpiThreads;
                nr[b] = -1;
                if (idx < BN * per_row) {
                  const int nrow = idx / per_row, rem = idx - nrow * per_row;
                  const int sb = rem / chunks, c = rem - sb * chunks;
                  if (s_slots[nrow] >= 0) {
                    nr[b] = nrow;
                    off[b] = sb * 256 + c;
                    const float* ur = a.u + (size_t)(t0 + nrow) * r_tot + u_off + sb * p.lora_sub + c * 8;
                    lo[b] = *reinterpret_cast<const float4*>(ur);
                    hi[b] = *reinterpret_cast<const float4*>(ur + 4);
                  }
                }
              }
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                if (nr[b] < 0) continue;
                const int nrow = nr[b], sb = off[b] >> 8, c = off[b] & 255;
                const int slot = s_slots[nrow];
                int sgi = 0;
                while (e_list[sgi] != slot) ++sgi;  // slot is in the list by construction
                const float sc = e_scale[sgi];
                const float f[8] = {lo[b].x * sc, lo[b].y * sc, lo[b].z * sc, lo[b].w * sc,
                                    hi[b].x * sc, hi[b].y * sc, hi[b].z * sc, hi[b].w * sc};
                const int sw = rb == 128 ? (nrow & 7) : rb == 64 ? ((nrow >> 1) & 3) : ((nrow >> 2) & 1);
                if (runs) {  // the adapter's own blocks only (block starts are multiples of 16 rows: same swizzle phase)
                  const int4 tb = e_tab[sgi];
                  *reinterpret_cast<uint4*>(s_cache + (size_t)(tb.z * p.n_sub + sb * tb.y + (nrow - tb.x)) * rb + ((c ^ sw) << 4)) = pack8(f);
                } else {
                  *reinterpret_cast<uint4*>(s_cache + (sgi * p.n_sub + sb) * BN * rb + nrow * rb + ((c ^ sw) << 4)) = pack8(f);
                }
              }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            epi_bar_sync();
            if (etid == 0) mbar_arrive(cache_full);
            e_key = tok_tile * 8 + mod;
          }
        }
      }

      // NormFuse producer: this CTA will finish the tile (whole tile, or first contributor of a split one), so the
      // residual values its epilogue adds are requested now, long before the accumulator is complete.
      float rs[32];
      float nw = 0.f;
      bool do_res = false;
      if constexpr (BN <= 32 && NF) {
        do_res = nf.res != nullptr && (full_seg || (int)blockIdx.x == (int)(((long long)sg.tile * p.k_blocks) / p.per_cta));
        if (do_res) {
#pragma unroll
          for (int i = 0; i < C::kChunk; ++i)
            rs[i] = (t0 + i < a.T && row < a.out) ? __ldcg(nf.res + (size_t)(t0 + i) * nf.ld_res + row) : 0.f;
          nw = row < a.out ? __bfloat162float(nf.norm_w[row]) : 0.f;
        }
      }

      // Adds the CUDA-core LoRA expand if any, applies SiLU*up, stores.  v[i] = (token t0+c0+i, row).
      auto finish = [&](float (&v)[32], int c0) {
        if (LM == 1) simt_lora_expand<BN>(a, v, c0, t0, row, r_tot, stage_u, s_slots, s_u);
        if constexpr (BN <= 32 && NF) {
          if (nf.sumsq_in != nullptr) {
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) v[i] *= s_rstd[c0 + i];
          }
          if (do_res) {
            float sq[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) sq[i] = 0.f;
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) {
              const int t = t0 + c0 + i;
              const bool live = t < a.T && row < a.out;
              const float xr = rs[i] + v[i];
              if (live) {
                nf.res[(size_t)t * nf.ld_res + row] = xr;
                sq[i] = xr * xr;
              }
              v[i] = xr * nw;
            }
            // sum over the warp's 32 rows, token by token: after the five exchange steps lane l holds token l's sum
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
              const bool up = (lane & off) != 0;
#pragma unroll
              for (int jj = 0; jj < off; ++jj) {
                const float send = up ? sq[jj] : sq[jj + off];
                const float keep = up ? sq[jj + off] : sq[jj];
                sq[jj] = keep + __shfl_xor_sync(0xffffffffu, send, off);
              }
            }
            s_red[q * 32 + lane] = sq[0];
            epi_bar_sync();
            if (etid < 32)
              nf.sumsq_out[(size_t)row_tile * 32 + etid] = (s_red[etid] + s_red[32 + etid]) + (s_red[64 + etid] + s_red[96 + etid]);
            epi_bar_sync();  // s_red is free again
          }
        }
        if (p.tma_store) {
          // registers -> shared memory [tokens][outputs of the tile] -> one TMA store (which also clips
          // tokens >= T and outputs >= out); far fewer instructions than 32 strided stores per thread
          if (etid == 0) bulk_wait_read0();  // the previous chunk's store has finished reading s_out
          epi_bar_sync();
          if (silu) {
            bf16* so = reinterpret_cast<bf16*>(s_out);
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) {
              const float other = __shfl_xor_sync(0xffffffffu, v[i], 8);
              if ((etid & 8) == 0) so[i * (BM / 2) + (etid >> 4) * 8 + (etid & 7)] = __float2bfloat16_rn(silu_mul(v[i], other));
            }
          } else if (out_f32) {
            float* so = reinterpret_cast<float*>(s_out);
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) so[i * BM + etid] = v[i];
          } else {
            bf16* so = reinterpret_cast<bf16*>(s_out);
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) so[i * BM + etid] = __float2bfloat16_rn(v[i]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          epi_bar_sync();
          if (etid == 0) tma_store_2d(&map_y, s_out, silu ? row_tile * (BM / 2) : row_tile * BM, t0 + c0);
          return;
        }
#pragma unroll
        for (int i = 0; i < C::kChunk; ++i) {
          const int t = t0 + c0 + i;
          const bool live = t < a.T && row < a.out;
          if (silu) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 8);
            if (live && (etid & 8) == 0) store_out(a, t, (row >> 4) * 8 + (row & 7), silu_mul(v[i], other));
          } else if (live) {
            store_out(a, t, row, v[i]);
          }
        }
      };

      // Split tile: who contributes, and is this CTA the one that finishes it?
      long long ts = 0, te = 0;
      int c_first = 0, c_last = 0;
      if (!full_seg) {
        ts = (long long)sg.tile * p.k_blocks;
        te = ts + p.k_blocks;
        c_first = (int)(ts / p.per_cta);
        c_last = (int)((te - 1) / p.per_cta);
      }
      const bool finisher = !full_seg && (int)blockIdx.x == c_first;
      // Single-chunk token tiles: the finisher collects the other contributors' partial sums NOW, while its own
      // last MMAs are still running (the contributors met this tile at the very start of their ranges, so their
      // partials have been in L2 for a long time), instead of after them in the kernel's tail.
      float pre[32];
      bool pre_have = true;
      if constexpr (BN <= 32) {
        if (finisher) {
          if (etid == 0) {
            const int need = c_last - c_first;
            bool got = false;
            for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
              int seen;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.tickets + c_first) : "memory");
              if (seen >= need) {
                got = true;
                break;
              }
              __nanosleep(64);
            }
            p.tickets[c_first] = 0;  // ready for the next call
            s_last = got ? 1 : 0;
            if (!got) atomicOr(p.status, 128);
          }
          epi_bar_sync();
          pre_have = s_last != 0;
#pragma unroll
          for (int i = 0; i < C::kChunk; ++i) pre[i] = 0.f;
          if (pre_have) {
            // CTA order: deterministic.  Two contributors' partials are requested together: each is a round trip to
            // L2 (or DRAM, behind the weight stream), and tiles of narrow projections have four or five of them.
            for (int cc = c_first + 1; cc <= c_last; cc += 2) {
              const float* ps = p.partials + ((size_t)cc * 2) * (size_t)(BN * BM);
              const bool two = cc + 1 <= c_last;
              float a0[C::kChunk], a1[C::kChunk];
#pragma unroll
              for (int i = 0; i < C::kChunk; ++i) a0[i] = __ldcg(ps + (size_t)i * BM + etid);
              if (two) {
#pragma unroll
                for (int i = 0; i < C::kChunk; ++i) a1[i] = __ldcg(ps + (size_t)2 * (BN * BM) + (size_t)i * BM + etid);
              }
#pragma unroll
              for (int i = 0; i < C::kChunk; ++i) pre[i] += a0[i];
              if (two) {
#pragma unroll
                for (int i = 0; i < C::kChunk; ++i) pre[i] += a1[i];
              }
            }
          }
          epi_bar_sync();  // s_last is reused by the next split segment
        }
      }

      if (!mbar_wait(&acc_full[buf], (j >> 1) & 1, &s_abort)) {
        if (!s_abort) {
          s_abort = 1;
          atomicOr(p.status, 4);
        }
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;

      if (full_seg) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
          if (BN >= 32) tmem_ld32(t_addr + c0, v); else tmem_ld16(t_addr + c0, v);
          if (c0 + 32 >= BN) {  // accumulator fully read: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
          finish(v, c0);
        }
      } else {
        // Split tile.  Contributors = the CTAs whose ranges meet [tile*k_blocks, (tile+1)*k_blocks).  The
        // first of them (the one holding the tile's first k-blocks) reaches this segment at the very end
        // of its range, after every other contributor has long passed theirs, so it is the one that
        // finishes the tile: the others publish an fp32 partial in scratch and bump the tile's counter;
        // the finisher waits (bounded) for the counter, adds the partials to its own accumulator in CTA
        // order -- deterministic -- and runs the epilogue.  It never writes a partial of its own.
        if (!finisher) {
          // slot 0 if this CTA's range starts inside the tile (always, except for c_first), kept general
          const bool starts_here = rg.it0 >= ts;
          float* part = p.partials + ((size_t)blockIdx.x * 2 + (starts_here ? 0 : 1)) * (size_t)(BN * BM);
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            float v[32];
            if (BN >= 32) tmem_ld32(t_addr + c0, v); else tmem_ld16(t_addr + c0, v);
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) part[(size_t)(c0 + i) * BM + etid] = v[i];
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          // the CTA-wide barrier orders every thread's partial stores before thread 0's release, which publishes
          // them (cumulatively) to the finisher's acquire: one fence instead of one per thread
          epi_bar_sync();
          if (etid == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.tickets + c_first) : "memory");
        } else if constexpr (BN <= 32) {
          float v[32];
          if (BN >= 32) tmem_ld32(t_addr, v); else tmem_ld16(t_addr, v);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
          if (pre_have) {
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) v[i] += pre[i];
            finish(v, 0);
          }
        } else {
          if (etid == 0) {
            const int need = c_last - c_first;
            bool got = false;
            for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
              int seen;
              asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(p.tickets + c_first) : "memory");
              if (seen >= need) {
                got = true;
                break;
              }
              __nanosleep(64);
            }
            p.tickets[c_first] = 0;  // ready for the next call
            s_last = got ? 1 : 0;
            if (!got) atomicOr(p.status, 128);
          }
          epi_bar_sync();
          const bool have = s_last != 0;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            float v[32];
            if (BN >= 32) tmem_ld32(t_addr + c0, v); else tmem_ld16(t_addr + c0, v);
            if (c0 + 32 >= BN) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
            if (have) {
              for (int cc = c_first + 1; cc <= c_last; ++cc) {
                const float* ps = p.partials + ((size_t)cc * 2) * (size_t)(BN * BM);
#pragma unroll
                for (int i = 0; i < C::kChunk; ++i) v[i] += __ldcg(ps + (size_t)(c0 + i) * BM + etid);
              }
              finish(v, c0);
            }
          }
          epi_bar_sync();  // s_last is reused by the next split segment
        }
      }
      ++j;
    }
  }

  // ---- teardown -----------------------------------------------------------------------------------------
  // epilogue thread 0 (warp 4, lane 0) issued the stores: shared memory must stay valid until they have
  // read it; their global writes complete with the grid
  if (p.tma_store && warp == 4 && lane == 0) bulk_wait_read0();
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    // give copies that may still be in flight a bounded time to land before the CTA exits
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
}

// ---- host side -------------------------------------------------------------------------------------
int pick_bn(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128; }

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
    return v > kMaxGrid ? kMaxGrid : v;
  }();
  return n;
}

struct Plan {
  int bn, row_tiles, tok_tiles, k_blocks, grid, per_cta, wave_gt, wave_full, wave_ch, wave_ch_last, wave_lanes;
};

// min_waves: whole-tile mode needs at least this many tiles per CTA, so that the unfilled last wave costs little.
Plan plan_for(int bn, int min_waves, int T, int in, int out) {
  Plan pl;
  pl.bn = bn;
  pl.row_tiles = (out + BM - 1) / BM;
  pl.tok_tiles = (T + pl.bn - 1) / pl.bn;
  pl.k_blocks = (in + BK - 1) / BK;
  const long long total = (long long)pl.row_tiles * pl.tok_tiles * pl.k_blocks;
  long long grid = sm_count();
  pl.wave_gt = pl.wave_full = pl.wave_ch = pl.wave_ch_last = pl.wave_lanes = 0;
  const long long n_tiles = (long long)pl.row_tiles * pl.tok_tiles;
  if (pl.tok_tiles >= 4 && n_tiles >= min_waves * grid) {
    // Waves of (token tiles x row tiles).
    static const int lane_form = [] {
      const char* e = getenv("MLORA_WAVE_LANES");
      return e ? atoi(e) : 1;
    }();
    if (lane_form) {
      // Lane form.  Token tiles per group: the group's token rows are what the CTAs re-read from L2 row tile after row
      // tile, so they should stay resident next to the weight tiles in flight (<= 48 MB of the 126 MB).  Among the
      // sizes that fit, the one with the fewest steps (groups x row tiles per lane); fewer groups on ties (each group
      // streams the weights once).
      long long best = -1;
      for (int d = 1; d <= 48 && d <= pl.tok_tiles && d <= (int)grid; ++d) {
        if (d > 1 && (double)d * pl.bn * in * 2.0 > 48e6) break;
        const int lanes = (int)grid / d;
        const int steps = (pl.row_tiles + lanes - 1) / lanes;
        const int groups = (pl.tok_tiles + d - 1) / d;
        const long long cost = (long long)groups * steps;
        if (best < 0 || cost <= best) {
          best = cost;
          pl.wave_gt = d;
          pl.wave_lanes = lanes;
          pl.wave_ch = steps;
          pl.wave_full = groups;
        }
      }
      pl.wave_ch_last = 0;
      pl.per_cta = pl.wave_full * pl.wave_ch * pl.k_blocks;
      pl.grid = (int)grid;
      return pl;
    }
    // Chunk form: the tiles of a group, token tile major / row tile minor, cut into equal contiguous chunks.  Token tiles
    // per group: the group's token rows should stay L2-resident (<= 56 MB), and row_tiles * group should fill whole
    // rounds of the grid (the slots beyond it idle); among the sizes that fit, the one that wastes the fewest slots.
    int gt = 1;
    double best = 2.0;
    for (int d = 1; d <= 48 && d <= pl.tok_tiles; ++d) {
      if (d > 1 && (double)d * pl.bn * in * 2.0 > 56e6) break;
      const long long tiles = (long long)pl.row_tiles * d;
      const long long slots = (tiles + grid - 1) / grid * grid;
      const double waste = (double)(slots - tiles) / (double)slots;
      if (waste <= best + 1e-9) {
        best = waste;
        gt = d;
      }
    }
    pl.wave_gt = gt;
    pl.wave_full = pl.tok_tiles / pl.wave_gt;
    const int gt_last = pl.tok_tiles - pl.wave_full * pl.wave_gt;
    pl.wave_ch = (int)(((long long)pl.row_tiles * pl.wave_gt + grid - 1) / grid);
    pl.wave_ch_last = (int)(((long long)pl.row_tiles * gt_last + grid - 1) / grid);
    pl.per_cta = (pl.wave_full * pl.wave_ch + pl.wave_ch_last) * pl.k_blocks;
    pl.grid = (int)grid;
    return pl;
  }
  // at least 4 k-blocks (64 KB of weights) per CTA, so tiny problems do not pay for 148 partial tiles
  if (grid > (total + 3) / 4) grid = (total + 3) / 4;
  if (grid < 1) grid = 1;
  pl.per_cta = (int)((total + grid - 1) / grid);
  pl.grid = (int)((total + pl.per_cta - 1) / pl.per_cta);
  return pl;
}

// 256-token tiles where whole tiles fill the grid at least three times over (prompt passes of thousands of rows): a
// 128 x 128 tile moves 64 KB through shared memory per 256 tensor-pipe cycles, twice what a shared memory delivers;
// 128 x 256 moves 96 KB per 512.  Switch: MLORA_TILE256=0 keeps 128-token tiles.
bool tile256_enabled() {
  static const bool on = [] {
    const char* e = getenv("MLORA_TILE256");
    return !(e && e[0] == '0');
  }();
  return on;
}

Plan make_plan(int T, int in, int out) {
  if (T >= 1024 && tile256_enabled()) {
    Plan big = plan_for(256, 3, T, in, out);
    if (big.wave_gt > 0) return big;
  }
  return plan_for(pick_bn(T), 8, T, in, out);
}

template <int BN>
int launch(const LinearArgs& a, const Plan& pl, void* work, cudaStream_t st) {
  using C = Cfg<BN>;
  CUtensorMap mw, mx;
  int rc = make_map(&mx, a.x, a.T, a.in, a.ldx, BN);
  if (rc) return rc;
  if (a.flags & MLORA_W_PACKED) {
    mw = mx;  // unused by the kernel
  } else {
    rc = make_map(&mw, a.W, a.out, a.in, a.in, BM);
    if (rc) return rc;
  }
  TcParams p;
  p.a = a;
  // LoRA expand: on the tensor cores when the rank pitch is 16/32/64/128 and every module boundary
  // is a multiple of the 128-row tile; else on CUDA cores in the epilogue (needs pitch <= 64)
  p.lora_mode = 0;
  p.lora_sub = 16;
  p.n_sub = 1;
  CUtensorMap mb = mw;
  if (a.u != nullptr) {
    bool aligned_mods = true;
    for (int m = 1; m < a.n_mod; ++m) aligned_mods = aligned_mods && (a.mod_off[m] % BM == 0);
    const bool pitch_ok = a.r_max == 16 || a.r_max == 32 || a.r_max == 64 || a.r_max == 128;
    if (pitch_ok && aligned_mods) {
      p.lora_mode = 2;
      p.lora_sub = a.r_max < 64 ? a.r_max : 64;
      p.n_sub = a.r_max / p.lora_sub;
      if (!(a.flags & MLORA_B_PACKED)) {
        rc = make_map(&mb, a.B_all, (long long)a.n_adapters * a.out, a.r_max, a.r_max, BM, p.lora_sub);
        if (rc) return rc;
      }
    } else {
      if (a.flags & MLORA_B_PACKED)
        return fail(MLORA_EINVAL, "linear: a packed B_all needs rank pitch 16/32/64/128 and tile-aligned modules");
      if (a.r_max > 64) return fail(MLORA_EINVAL, "linear: rank pitch %d needs tile-aligned modules", a.r_max);
      p.lora_mode = 1;
    }
  }
  p.k_blocks = pl.k_blocks;
  p.row_tiles = pl.row_tiles;
  p.n_tiles = pl.row_tiles * pl.tok_tiles;
  p.tok_tiles = pl.tok_tiles;
  p.wave_gt = pl.wave_gt;
  p.wave_full = pl.wave_full;
  p.wave_ch = pl.wave_ch;
  p.wave_ch_last = pl.wave_ch_last;
  p.wave_lanes = pl.wave_lanes;
  p.per_cta = pl.per_cta;
  // output through TMA when the tensor satisfies its alignment rules (16-byte base and row pitch)
  CUtensorMap my = mx;
  {
    const bool f32 = (a.flags & MLORA_OUT_F32) != 0, silu = (a.flags & MLORA_SILU_MUL) != 0;
    const int es = f32 ? 4 : 2, cols = silu ? a.out / 2 : a.out;
    p.tma_store = !(BN >= 128 && f32) && aligned16(a.y) && (a.ldy * es) % 16 == 0 && (cols * es) % 16 == 0;
    if (p.tma_store) {
      rc = make_out_map(&my, a.y, a.T, cols, a.ldy, BN < 32 ? BN : 32, silu ? BM / 2 : BM, f32);
      if (rc) return rc;
    }
  }
  p.prefetch = 0;  // measured: an L2 prefetch stream ahead of the ring slows the kernel down on B200
  p.status = (int32_t*)work;
  p.tickets = (int32_t*)((uint8_t*)work + kHeaderBytes);
  p.partials = (float*)((uint8_t*)work + kHeaderBytes + kMaxGrid * 4);
  // the shared-memory opt-in is a per-device attribute of each instantiation
  static std::atomic<unsigned long long> attr_done{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!((attr_done.load(std::memory_order_acquire) >> (dev & 63)) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<BN, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(linear_tc_kernel<BN, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(linear_tc_kernel<BN, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return fail(MLORA_ECUDA, "linear: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  if constexpr (BN <= 32) {
    if (a.nf.res != nullptr || a.nf.sumsq_in != nullptr) {
      if (p.lora_mode == 1) return fail(MLORA_EINVAL, "linear_norm: the LoRA expand of this call runs on CUDA cores (rank pitch / module alignment)");
      static std::atomic<unsigned long long> nf_attr_done{0};
      if (!((nf_attr_done.load(std::memory_order_acquire) >> (dev & 63)) & 1ull)) {
        cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<BN, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(linear_tc_kernel<BN, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return fail(MLORA_ECUDA, "linear: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        nf_attr_done.fetch_or(1ull << (dev & 63), std::memory_order_release);
      }
      if (p.lora_mode == 2 || (a.flags & MLORA_SHARE_LORA_KERNEL))
        launch_pdl_if(pdl_enabled_gemm(), linear_tc_kernel<BN, 2, true>, pl.grid, kThreads, C::kSmemBytes, st, mw, mx, mb, my, p);
      else
        launch_pdl_if(pdl_enabled_gemm(), linear_tc_kernel<BN, 0, true>, pl.grid, kThreads, C::kSmemBytes, st, mw, mx, mb, my, p);
      count_launch();
      MLORA_CHECK_LAUNCH("linear_tc_kernel");
      return MLORA_OK;
    }
  }
  if (p.lora_mode == 1)
    launch_pdl_if(pdl_enabled_gemm(), linear_tc_kernel<BN, 1>, pl.grid, kThreads, C::kSmemBytes, st, mw, mx, mb, my, p);
  else if (p.lora_mode == 2 || (a.flags & MLORA_SHARE_LORA_KERNEL))
    launch_pdl_if(pdl_enabled_gemm(), linear_tc_kernel<BN, 2>, pl.grid, kThreads, C::kSmemBytes, st, mw, mx, mb, my, p);
  else
    launch_pdl_if(pdl_enabled_gemm(), linear_tc_kernel<BN, 0>, pl.grid, kThreads, C::kSmemBytes, st, mw, mx, mb, my, p);
  count_launch();
  MLORA_CHECK_LAUNCH("linear_tc_kernel");
  return MLORA_OK;
}

// Repacks W [out, in] into tiles [row_tile][k_block][128 rows][64 k] whose bytes are the
// shared-memory image the MMA reads: row r of a tile at r*128 bytes, its 16-byte chunk c at
// ((c ^ (r & 7)) * 16) (128-byte swizzle).  Rows / columns past the matrix are zero.
__global__ void __launch_bounds__(256) pack_weight_kernel(const bf16* __restrict__ W, int out, int in, int k_blocks,
                                                          uint4* __restrict__ Wp) {
  const size_t tile = blockIdx.x;  // row_tile * k_blocks + kb
  const int row_tile = (int)(tile / k_blocks), kb = (int)(tile % k_blocks);
  for (int idx = threadIdx.x; idx < BM * 8; idx += blockDim.x) {
    const int r = idx >> 3, c = idx & 7;
    const int row = row_tile * BM + r, k = kb * BK + c * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < out && k < in) v = *reinterpret_cast<const uint4*>(W + (size_t)row * in + k);  // in % 8 == 0
    Wp[tile * (BM * 8) + r * 8 + (c ^ (r & 7))] = v;
  }
}

// Repacks B_all [N, out, r_max] into tiles [slot][row_tile][sub-block][128 rows][lora_sub] whose bytes
// are the shared-memory image of a LoRA stage's A operand: row r at r*rb bytes (rb = 2*lora_sub), its
// 16-byte chunk c at ((c ^ swizzle(r)) * 16), swizzle span = rb.  Rows past `out` are zero.
__global__ void __launch_bounds__(256) pack_lora_b_kernel(const bf16* __restrict__ B, int out, int r_max,
                                                          int row_tiles, int lora_sub, int n_sub,
                                                          uint4* __restrict__ Bp) {
  const size_t tile = blockIdx.x;  // (slot * row_tiles + row_tile) * n_sub + sb
  const int sb = (int)(tile % n_sub);
  const size_t sr = tile / n_sub;
  const int row_tile = (int)(sr % row_tiles), slot = (int)(sr / row_tiles);
  const int chunks = lora_sub / 8, rb = lora_sub * 2;
  for (int idx = threadIdx.x; idx < BM * chunks; idx += blockDim.x) {
    const int r = idx / chunks, c = idx - r * chunks;
    const int row = row_tile * BM + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < out) v = *reinterpret_cast<const uint4*>(B + ((size_t)slot * out + row) * r_max + sb * lora_sub + c * 8);
    const int sw = rb == 128 ? (r & 7) : rb == 64 ? ((r >> 1) & 3) : ((r >> 2) & 1);
    Bp[tile * (BM * chunks) + r * chunks + (c ^ sw)] = v;
  }
}

}  // namespace

size_t packed_lora_b_bytes(int n_adapters, int out, int r_max) {
  return (size_t)n_adapters * ((out + BM - 1) / BM) * BM * r_max * 2;
}

int launch_pack_lora_b(const void* B, int n_adapters, int out, int r_max, void* Bp, cudaStream_t st) {
  if (!(r_max == 16 || r_max == 32 || r_max == 64 || r_max == 128))
    return fail(MLORA_EINVAL, "pack_lora_b: rank pitch must be 16, 32, 64 or 128 (got %d)", r_max);
  const int lora_sub = r_max < 64 ? r_max : 64, n_sub = r_max / lora_sub;
  const int row_tiles = (out + BM - 1) / BM;
  const long long tiles = (long long)n_adapters * row_tiles * n_sub;
  if (tiles > 2147483647ll) return fail(MLORA_ESIZE, "pack_lora_b: stack too large");
  pack_lora_b_kernel<<<(unsigned)tiles, 256, 0, st>>>((const bf16*)B, out, r_max, row_tiles, lora_sub, n_sub, (uint4*)Bp);
  count_launch();
  MLORA_CHECK_LAUNCH("pack_lora_b_kernel");
  return MLORA_OK;
}

size_t packed_weight_bytes(int out, int in) {
  return (size_t)((out + BM - 1) / BM) * ((in + BK - 1) / BK) * (BM * BK * 2);
}

int launch_pack_weight(const void* W, int out, int in, void* Wp, cudaStream_t st) {
  const int k_blocks = (in + BK - 1) / BK;
  const long long tiles = (long long)((out + BM - 1) / BM) * k_blocks;
  if (tiles > 2147483647ll) return fail(MLORA_ESIZE, "pack_weight: matrix too large");
  pack_weight_kernel<<<(unsigned)tiles, 256, 0, st>>>((const bf16*)W, out, in, k_blocks, (uint4*)Wp);
  count_launch();
  MLORA_CHECK_LAUNCH("pack_weight_kernel");
  return MLORA_OK;
}

bool linear_tc_supported(const LinearArgs& a) {
  // TMA needs 16-byte aligned bases and row pitches; everything else (ragged K, out, T) is handled by
  // zero-filled out-of-bounds boxes and masked stores.
  const long long tiles = (long long)((a.out + BM - 1) / BM) * ((a.T + 127) / 128);
  return aligned16(a.x) && aligned16(a.W) && (a.ldx * 2) % 16 == 0 && (a.in * 2) % 16 == 0 && (a.u == nullptr || a.r_max % 8 == 0) &&
         (a.u == nullptr || a.r_max <= 64 || a.r_max == 128) &&
         tiles * ((a.in + BK - 1) / BK) < 2000000000ll;
}

// How a projection of this shape is dealt to the CTAs (host-side planning only; no device work).
void linear_tc_plan(int T, int in, int out, int32_t* v) {
  const Plan pl = make_plan(T, in, out);
  v[0] = pl.bn;
  v[1] = pl.grid;
  v[2] = pl.row_tiles;
  v[3] = pl.tok_tiles;
  v[4] = pl.k_blocks;
  v[5] = pl.per_cta;
  v[6] = pl.wave_gt;
  v[7] = pl.wave_lanes;
  v[8] = pl.wave_ch;
  v[9] = pl.wave_full;
  v[10] = pl.wave_ch_last;
  v[11] = 0;
}

size_t linear_tc_workspace(int T, int in, int out) {
  const int bn = T > 0 ? pick_bn(T) : 16;
  return kHeaderBytes + kMaxGrid * 4 + (size_t)kMaxGrid * 2 * bn * BM * sizeof(float);
}

int launch_linear_tc(const LinearArgs& a, void* work, size_t work_bytes, cudaStream_t st) {
  const size_t need = linear_tc_workspace(a.T, a.in, a.out);
  if (work_bytes < need) return fail(MLORA_ESIZE, "linear: workspace of %zu bytes needed, %zu given", need, work_bytes);
  Plan pl = make_plan(a.T, a.in, a.out);
  switch (pl.bn) {
    case 16: return launch<16>(a, pl, work, st);
    case 32: return launch<32>(a, pl, work, st);
    case 64: return launch<64>(a, pl, work, st);
    case 256: return launch<256>(a, pl, work, st);
    default: return launch<128>(a, pl, work, st);
  }
}

}  // namespace mlora
