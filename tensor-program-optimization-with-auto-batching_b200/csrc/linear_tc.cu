// Weight-streaming projection kernel on the 5th-generation tensor cores (tcgen05 + TMEM), fed by
// TMA.  y[T,out] = x[T,in] W[out,in]^T with T small (decode) or tiled (prefill): the weight tile
// is the 128-row M operand, the token rows are the N operand ("swap-AB"), so the 128 x BN fp32
// accumulator lives in BN TMEM columns and one thread issues all MMAs.
//
// CTA = 128 threads: thread 0 of warp 0 drives TMA, thread 0 of warp 1 issues tcgen05.mma, then
// all four warps run the epilogue (one TMEM lane = one output row per thread).
// Grid = (row tiles of 128, token tiles of BN, K splits).  With K splits > 1 each CTA writes its
// fp32 partial tile to scratch and the last CTA to arrive (atomic ticket) sums the partials in
// split order -- deterministic -- and runs the epilogue (LoRA expand, SiLU*up, store).
//
// Every wait on an mbarrier is bounded; on expiry the CTA records a code in the status word at
// the start of the scratch buffer and leaves without touching the output.
#include <cuda.h>

#include "linear.cuh"

namespace mlora {
namespace {

constexpr int BM = 128;        // weight rows per CTA (MMA M)
constexpr int BK = 64;         // K elements per stage = one 128-byte swizzle span
constexpr int kHeaderBytes = 256;  // status word + padding at the start of the scratch buffer
constexpr int kMaxTickets = 16384; // split-K arrival counters live in a fixed region after the header, so
                                   // that calls of different shapes sharing one scratch buffer never
                                   // overlay partial sums on counters
constexpr uint32_t kSpinLimit = 1u << 24;

struct TcParams {
  LinearArgs a;
  int k_blocks;       // ceil(in / BK)
  int kb_per_split;
  int n_splits;
  int32_t* status;    // scratch[0]
  int32_t* tickets;   // [row_tiles * token_tiles]
  float* partials;    // [row_tiles * token_tiles][n_splits][BN][BM]
};

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait; false = gave up (or another role raised `abort`).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((i & 1023) == 1023 && *abort) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 lanes x 32 columns of fp32: register i of lane l = TMEM[lane_base + l][col + i].
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024
// bytes apart.  Field layout of the sm_100 shared-memory matrix descriptor: start address >> 4 in
// bits [0,14), leading byte offset >> 4 in [16,30) (unused for swizzled K-major, set to 1), stride
// byte offset >> 4 in [32,46), descriptor version 1 in [46,48), swizzle mode in [61,64) (2 = 128 B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor, kind::f16: D fp32 (bits [4,6) = 1), A and B bf16 ([7,10) = [10,13) = 1),
// both K-major (bits 15,16 = 0), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int BN>
struct Cfg {
  static constexpr int kStageBytes = BM * BK * 2 + BN * BK * 2;
  static constexpr int kBudget = BN <= 64 ? 100 * 1024 : 200 * 1024;  // <= 64 tokens: two CTAs per SM
  static constexpr int kStages = (kBudget / kStageBytes) > 8 ? 8 : (kBudget / kStageBytes);
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
};

template <int BN>
__global__ void __launch_bounds__(128) linear_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                        const __grid_constant__ CUtensorMap map_x, TcParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + C::kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* accum_bar = empty_bar + C::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  __shared__ int s_abort;
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_tile = blockIdx.x, tok_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(kb0 + p.kb_per_split, p.k_blocks);
  const int n_kb = kb1 - kb0;  // >= 1 by construction of the grid

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ------------------------------------------------------------------------------
    for (int i = 0; i < n_kb; ++i) {
      const int s = i % C::kStages, round = i / C::kStages;
      if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &s_abort)) {
        s_abort = 1;
        atomicOr(p.status, 1);
        break;
      }
      uint8_t* st = tiles + s * C::kStageBytes;
      mbar_expect_tx(&full_bar[s], C::kStageBytes);
      tma_load_2d(st, &map_w, (kb0 + i) * BK, row_tile * BM, &full_bar[s]);
      tma_load_2d(st + BM * BK * 2, &map_x, (kb0 + i) * BK, tok_tile * BN, &full_bar[s]);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer --------------------------------------------------------------------------------
    constexpr uint32_t idesc = make_idesc(BM, BN < 16 ? 16 : BN);
    bool ok = true;
    for (int i = 0; i < n_kb && ok; ++i) {
      const int s = i % C::kStages, round = i / C::kStages;
      if (!mbar_wait(&full_bar[s], round & 1, &s_abort)) {
        s_abort = 1;
        atomicOr(p.status, 2);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t wa = smem_u32(tiles + s * C::kStageBytes);
      const uint64_t adesc = make_smem_desc(wa);
      const uint64_t bdesc = make_smem_desc(wa + BM * BK * 2);
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) {
        // advancing 16 elements (32 bytes) along K inside the swizzle span = +2 in the address field
        umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0);
      }
      umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
    }
    if (ok) umma_commit(accum_bar);
  }

  // ---- epilogue: all 128 threads -----------------------------------------------------------------------
  __syncwarp();
  bool have_acc = mbar_wait(accum_bar, 0, &s_abort);
  if (!have_acc && !s_abort) {
    s_abort = 1;
    atomicOr(p.status, 4);
  }
  tc_fence_after();
  __syncthreads();
  const bool aborted = s_abort != 0;

  const LinearArgs& a = p.a;
  const int row = row_tile * BM + tid;        // output feature of this thread
  const int t0 = tok_tile * BN;
  const uint32_t t_lane = tmem_base + ((uint32_t)(warp * 32) << 16);
  const bool silu = (a.flags & MLORA_SILU_MUL) != 0;

  auto finish = [&](const float (&v)[32], int c0, int n) {
    // v[i] = base projection of (token t0+c0+i, feature row)
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i < n) {
        const int t = t0 + c0 + i;
        const bool live = t < a.T && row < a.out;
        float val = v[i];
        if (live) val += lora_expand(a, t, row);
        if (silu) {
          const float other = __shfl_xor_sync(0xffffffffu, val, 8);
          if (live && (tid & 8) == 0) store_out(a, t, (row >> 4) * 8 + (row & 7), silu_mul(val, other));
        } else if (live) {
          store_out(a, t, row, val);
        }
      }
    }
  };

  if (!aborted) {
    if (p.n_splits == 1) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        if (BN >= 32) tmem_ld32(t_lane + c0, v); else tmem_ld16(t_lane + c0, v);
        finish(v, c0, BN < 32 ? BN : 32);
      }
    } else {
      const size_t tile_id = (size_t)tok_tile * gridDim.x + row_tile;
      float* part = p.partials + (tile_id * p.n_splits + split) * (size_t)(BN * BM);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        float v[32];
        if (BN >= 32) tmem_ld32(t_lane + c0, v); else tmem_ld16(t_lane + c0, v);
#pragma unroll
        for (int i = 0; i < (BN < 32 ? BN : 32); ++i) part[(size_t)(c0 + i) * BM + tid] = v[i];
      }
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int ticket = atomicAdd(&p.tickets[tile_id], 1);
        s_last = ticket == p.n_splits - 1;
        if (s_last) p.tickets[tile_id] = 0;  // ready for the next call
      }
      __syncthreads();
      if (s_last) {
        __threadfence();
        const float* base = p.partials + tile_id * p.n_splits * (size_t)(BN * BM);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
          for (int s = 0; s < p.n_splits; ++s) {
            const float* ps = base + (size_t)s * (BN * BM);
#pragma unroll
            for (int i = 0; i < (BN < 32 ? BN : 32); ++i) v[i] += __ldcg(ps + (size_t)(c0 + i) * BM + tid);
          }
          finish(v, c0, BN < 32 ? BN : 32);
        }
      }
    }
  } else {
    // give copies that may still be in flight a bounded time to land before the CTA exits
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
}

// ---- host side -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return (EncodeTiledFn)f;
  }();
  return fn;
}

// 2-D bf16 tensor [rows, cols] with row pitch ld elements; box = [box_rows, 64 cols], 128-byte swizzle.
int make_map(CUtensorMap* m, const void* ptr, int rows, int cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MLORA_ECUDA, "linear: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MLORA_ECUDA, "linear: cuTensorMapEncodeTiled failed with %d", (int)r);
  return MLORA_OK;
}

int pick_bn(int T) { return T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : 128; }

struct Plan {
  int bn, row_tiles, tok_tiles, k_blocks, n_splits, kb_per_split;
};

Plan make_plan(int T, int in, int out) {
  Plan pl;
  pl.bn = pick_bn(T);
  pl.row_tiles = (out + BM - 1) / BM;
  pl.tok_tiles = (T + pl.bn - 1) / pl.bn;
  pl.k_blocks = (in + BK - 1) / BK;
  // enough CTAs to put two on every SM, but at least 4 K blocks (32 KB of weights) per CTA
  const int base = pl.row_tiles * pl.tok_tiles;
  int s = (2 * 148 + base - 1) / base;
  const int max_s = pl.k_blocks / 4 > 0 ? pl.k_blocks / 4 : 1;
  if (s > max_s) s = max_s;
  if (s > 16) s = 16;
  if (s < 1 || base > kMaxTickets) s = 1;
  pl.kb_per_split = (pl.k_blocks + s - 1) / s;
  pl.n_splits = (pl.k_blocks + pl.kb_per_split - 1) / pl.kb_per_split;  // no empty split
  return pl;
}

template <int BN>
int launch(const LinearArgs& a, const Plan& pl, void* work, cudaStream_t st) {
  using C = Cfg<BN>;
  CUtensorMap mw, mx;
  int rc = make_map(&mw, a.W, a.out, a.in, a.in, BM);
  if (rc) return rc;
  rc = make_map(&mx, a.x, a.T, a.in, a.ldx, BN);
  if (rc) return rc;
  TcParams p;
  p.a = a;
  p.k_blocks = pl.k_blocks;
  p.kb_per_split = pl.kb_per_split;
  p.n_splits = pl.n_splits;
  p.status = (int32_t*)work;
  p.tickets = (int32_t*)((uint8_t*)work + kHeaderBytes);
  p.partials = (float*)((uint8_t*)work + kHeaderBytes + kMaxTickets * 4);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kSmemBytes);
    if (e != cudaSuccess) return fail(MLORA_ECUDA, "linear: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  dim3 grid(pl.row_tiles, pl.tok_tiles, pl.n_splits);
  linear_tc_kernel<BN><<<grid, 128, C::kSmemBytes, st>>>(mw, mx, p);
  count_launch();
  MLORA_CHECK_LAUNCH("linear_tc_kernel");
  return MLORA_OK;
}

}  // namespace

bool linear_tc_supported(const LinearArgs& a) {
  // TMA needs 16-byte aligned bases and row pitches; everything else (ragged K, out, T) is handled by
  // zero-filled out-of-bounds boxes and masked stores.
  return aligned16(a.x) && aligned16(a.W) && (a.ldx * 2) % 16 == 0 && (a.in * 2) % 16 == 0 &&
         (size_t)((a.out + BM - 1) / BM) <= 2147483647u && ((a.T + 127) / 128) <= 65535;
}

size_t linear_tc_workspace(int T, int in, int out) {
  if (T <= 0 || in <= 0 || out <= 0) return kHeaderBytes + kMaxTickets * 4;
  Plan pl = make_plan(T, in, out);
  const size_t n_tiles = (size_t)pl.row_tiles * pl.tok_tiles;
  size_t bytes = kHeaderBytes + kMaxTickets * 4;
  if (pl.n_splits > 1) bytes += n_tiles * pl.n_splits * (size_t)pl.bn * BM * sizeof(float);
  return bytes;
}

int launch_linear_tc(const LinearArgs& a, void* work, size_t work_bytes, cudaStream_t st) {
  const size_t need = linear_tc_workspace(a.T, a.in, a.out);
  if (work_bytes < need) return fail(MLORA_ESIZE, "linear: workspace of %zu bytes needed, %zu given", need, work_bytes);
  Plan pl = make_plan(a.T, a.in, a.out);
  switch (pl.bn) {
    case 16: return launch<16>(a, pl, work, st);
    case 32: return launch<32>(a, pl, work, st);
    case 64: return launch<64>(a, pl, work, st);
    default: return launch<128>(a, pl, work, st);
  }
}

}  // namespace mlora
