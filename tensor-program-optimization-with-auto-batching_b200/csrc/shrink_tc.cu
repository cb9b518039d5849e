// LoRA shrink at prefill sizes as a segmented grouped GEMM on the 5th-generation tensor cores
// (tcgen05 + TMEM), fed by TMA:   u[t, :] = A_all[slot[t]] (r_tot x in) . x[t, :]
//
// One CTA per tile of 128 token rows.  The token tile is the M operand (128 TMEM lanes = 128 tokens);
// for every DISTINCT adapter among the tile's rows the adapter's A matrix (r_tot rows, padded to a
// multiple of 16) is an N operand with its own accumulator columns, so a tile whose rows all use one
// adapter (the usual case: prompt rows are contiguous per request) costs one pass over x, and a mixed
// tile costs one extra MMA group per further adapter, not per row.  Rows pick their adapter's columns
// in the output write.  When the distinct adapters of a tile need more than the accumulator / stage
// budget they are processed in passes, each re-streaming the token tile (it is L2 resident).
//
// 192 threads: warp 0 = TMA producer (one thread), warp 1 = MMA issuer (one thread), warps 2..5 =
// output (one TMEM lane = one token row per thread).  Every wait is bounded; when one expires the CTA
// stops, writes NaN to its rows of u (so the failure cannot go unnoticed downstream) and leaves after
// its copies in flight have landed and its TMEM is freed.
#include <stdlib.h>

#include <atomic>

#include "linear.cuh"
#include "tc_ptx.cuh"

namespace mlora {
namespace {

constexpr int kTok = 128;           // token rows per CTA (MMA M)
constexpr int kShrinkThreads = 192;
constexpr int kXTile = kTok * BK * 2;  // 16 KB
constexpr int kMaxStages = 12;

struct ShrinkParams {
  const int32_t* slots;
  float* u;
  int T, r_tot, n_pad, n_adapters, k_blocks;
  int segs_per_pass;  // adapters whose accumulators / operand tiles fit at once
  int ring_bytes, tmem_cols;
};

__global__ void __launch_bounds__(kShrinkThreads, 1) lora_shrink_tc_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                           const __grid_constant__ CUtensorMap map_a,
                                                                           ShrinkParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full, acc_empty;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_tok[kTok];   // slot of each row (-1: no adapter / beyond T)
  __shared__ int s_seg[kTok];   // index of the row's adapter in s_list
  __shared__ int s_list[kTok];  // distinct adapters in order of first appearance
  __shared__ int s_nseg, s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t0 = blockIdx.x * kTok;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_full, 1);
    mbar_init(&acc_empty, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&map_x);
    tma_prefetch_desc(&map_a);
  }
  if (warp == 1) tmem_alloc(&tmem_slot, p.tmem_cols);
  pdl_launch_dependents();
  pdl_wait();
  if (tid < kTok) {
    const int t = t0 + tid;
    int s = t < p.T ? p.slots[t] : -1;
    if (s >= p.n_adapters) s = -1;
    s_tok[tid] = s;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {  // distinct adapters of the tile
    int n = 0;
    for (int base = 0; base < kTok; base += 32) {
      const int s = s_tok[base + lane];
      bool fresh = s >= 0;
      for (int j = 0; j < n; ++j) fresh = fresh && s_list[j] != s;
      const unsigned same = __match_any_sync(0xffffffffu, s);
      const bool first = fresh && (__ffs(same) - 1 == lane);
      const unsigned b = __ballot_sync(0xffffffffu, first);
      if (first) s_list[n + __popc(b & ((1u << lane) - 1u))] = s;
      n += __popc(b);
      __syncwarp();
    }
    if (lane == 0) s_nseg = n;
  }
  __syncthreads();
  const int n_seg = s_nseg;
  if (tid < kTok) {
    const int s = s_tok[tid];
    int j = -1;
    if (s >= 0)
      for (j = 0; s_list[j] != s; ++j) {
      }
    s_seg[tid] = j;
  }
  __syncthreads();
  const uint32_t tmem_base = tmem_slot;
  const int n_pass = (n_seg + p.segs_per_pass - 1) / p.segs_per_pass;
  const int a_tile = p.n_pad * 128;  // bytes of one adapter's operand tile in a stage
  // A stage holds the token tile and the operand tiles of the adapters THIS tile has (usually one: prompt rows of a
  // request are contiguous), so the ring is as deep as the shared memory allows: the kernel is a chain of L2 round trips
  // per k-block, and the number of stages in flight is its throughput.
  const int nj_max = max(1, min(n_seg, p.segs_per_pass));
  const int stage_bytes = kXTile + ((nj_max * a_tile + 1023) & ~1023);
  const int stages = min(kMaxStages, p.ring_bytes / stage_bytes);

  if (warp == 0 && lane == 0) {
    // ---- producer: token tile + the pass's adapter tiles per k-block ----
    int g = 0;
    bool ok = true;
    for (int ps = 0; ps < n_pass && ok; ++ps) {
      const int j0 = ps * p.segs_per_pass, nj = min(p.segs_per_pass, n_seg - j0);
      for (int kb = 0; kb < p.k_blocks; ++kb, ++g) {
        const int s = g % stages, round = g / stages;
        if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &s_abort)) {
          s_abort = 1;
          ok = false;
          break;
        }
        uint8_t* st = ring + (size_t)s * stage_bytes;
        mbar_expect_tx(&full_bar[s], (uint32_t)(kXTile + nj * a_tile));
        tma_load_2d(st, &map_x, kb * BK, t0, &full_bar[s]);
        for (int j = 0; j < nj; ++j)
          tma_load_2d(st + kXTile + j * a_tile, &map_a, kb * BK, s_list[j0 + j] * p.r_tot, &full_bar[s]);
      }
    }
    if (!ok) {
      // copies already issued still land in this CTA's shared memory: wait for them (bounded) before leaving
      int dummy = 0;
      for (int back = 1; back <= stages && back <= g; ++back) {
        const int gi = g - back;
        mbar_wait(&full_bar[gi % stages], (gi / stages) & 1, &dummy);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    const uint32_t idesc = make_idesc(kTok, p.n_pad);
    int g = 0;
    bool ok = true;
    for (int ps = 0; ps < n_pass && ok; ++ps) {
      const int j0 = ps * p.segs_per_pass, nj = min(p.segs_per_pass, n_seg - j0);
      if (ps > 0) {  // the output warps have drained the accumulators of the previous pass
        if (!mbar_wait(&acc_empty, (ps - 1) & 1, &s_abort)) {
          s_abort = 1;
          break;
        }
        tc_fence_after();
      }
      for (int kb = 0; kb < p.k_blocks; ++kb, ++g) {
        const int s = g % stages, round = g / stages;
        if (!mbar_wait(&full_bar[s], round & 1, &s_abort)) {
          s_abort = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t st = smem_u32(ring + (size_t)s * stage_bytes);
        const uint64_t adesc = make_smem_desc(st);
        for (int j = 0; j < nj; ++j) {
          const uint64_t bdesc = make_smem_desc(st + kXTile + j * a_tile);
          const uint32_t d = tmem_base + (uint32_t)(j * p.n_pad);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) umma_bf16(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      if (ok) umma_commit(&acc_full);
    }
  } else if (warp >= 2) {
    // ---- output: row i of the tile = TMEM lane i ----
    const int row = (warp & 3) * 32 + lane, t = t0 + row;
    const int my = s_seg[row];
    float* ur = p.u + (size_t)t * p.r_tot;
    if (t < p.T && my < 0)
      for (int c = 0; c < p.r_tot; c += 4) *reinterpret_cast<float4*>(ur + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    bool ok = true;
    for (int ps = 0; ps < n_pass && ok; ++ps) {
      const int j0 = ps * p.segs_per_pass, nj = min(p.segs_per_pass, n_seg - j0);
      int w = 1;
      if (lane == 0) w = mbar_wait(&acc_full, ps & 1, &s_abort) ? 1 : 0;
      w = __shfl_sync(0xffffffffu, w, 0);
      if (!w) {
        s_abort = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      for (int j = 0; j < nj; ++j) {
        const bool mine = my == j0 + j;
        if (!__any_sync(0xffffffffu, mine)) continue;  // warp-uniform: TMEM loads are warp-collective
        const uint32_t taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(j * p.n_pad);
        for (int c0 = 0; c0 < p.r_tot; c0 += 16) {
          float v[32];
          tmem_ld16(taddr + c0, v);
          if (mine && t < p.T) {
#pragma unroll
            for (int c = 0; c < 16; c += 4)
              if (c0 + c < p.r_tot) *reinterpret_cast<float4*>(ur + c0 + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty);
    }
  }
  __syncthreads();
  if (s_abort && warp >= 2) {
    const int t = t0 + (warp & 3) * 32 + lane;
    if (t < p.T)
      for (int c = 0; c < p.r_tot; ++c) p.u[(size_t)t * p.r_tot + c] = __int_as_float(0x7fc00000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, p.tmem_cols);
}

}  // namespace

bool lora_shrink_tc_supported(const void* x, int64_t ldx, const void* A_all, const float* u, int T, int in, int r_tot) {
  // worth it from a few token tiles on; below that the warp-per-(row, rank) kernel is latency bound anyway
  return T >= 256 && r_tot % 8 == 0 && r_tot <= 256 && in % 8 == 0 && ldx % 8 == 0 && aligned16(x) && aligned16(A_all) &&
         aligned16(u);
}

int launch_lora_shrink_tc(const void* x, int64_t ldx, const void* A_all, const int32_t* slots, int n_adapters, int T,
                          int in, int r_tot, float* u, cudaStream_t st) {
  ShrinkParams p;
  p.slots = slots;
  p.u = u;
  p.T = T;
  p.r_tot = r_tot;
  p.n_pad = (r_tot + 15) / 16 * 16;
  p.n_adapters = n_adapters;
  p.k_blocks = (in + BK - 1) / BK;
  p.segs_per_pass = 256 / p.n_pad;  // <= 32 KB of adapter tiles per stage, <= 256 accumulator columns
  if (p.segs_per_pass < 1) p.segs_per_pass = 1;
  // the ring: whole stages of the largest kind (all segs_per_pass operand tiles), at least two, within 200 KB
  const int stage_max = kXTile + ((p.segs_per_pass * p.n_pad * 128 + 1023) & ~1023);
  int n_max = (200 * 1024) / stage_max;
  if (n_max < 2) n_max = 2;
  p.ring_bytes = n_max * stage_max > 200 * 1024 ? n_max * stage_max : 200 * 1024;
  int cols = 32;
  while (cols < p.segs_per_pass * p.n_pad) cols *= 2;
  p.tmem_cols = cols;
  CUtensorMap mx, ma;
  int rc = make_map(&mx, x, T, in, ldx, kTok);
  if (rc) return rc;
  rc = make_map(&ma, A_all, (long long)n_adapters * r_tot, in, in, p.n_pad);
  if (rc) return rc;
  const size_t smem = (size_t)p.ring_bytes + 1024;
  static std::atomic<unsigned long long> attr_done{0};  // per-device attribute
  int dev = 0;
  cudaGetDevice(&dev);
  if (!((attr_done.load(std::memory_order_acquire) >> (dev & 63)) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(lora_shrink_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) return fail(MLORA_ECUDA, "lora_shrink: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  launch_pdl_if(pdl_enabled_shrink(), lora_shrink_tc_kernel, dim3((T + kTok - 1) / kTok), dim3(kShrinkThreads), smem, st, mx, ma, p);
  count_launch();
  MLORA_CHECK_LAUNCH("lora_shrink_tc_kernel");
  return MLORA_OK;
}

}  // namespace mlora
