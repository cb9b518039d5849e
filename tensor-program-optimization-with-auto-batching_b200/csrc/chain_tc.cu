// A chain of decode-size projections in ONE persistent launch: o -> (+residual, RMSNorm) -> gate|up (SiLU) ->
// down -> (+residual, RMSNorm, q/k/v shrink) -> q/k/v, i.e. everything between two attention calls of the
// decoder (tvm/llama_auto_batcher/llama_for_causal_lm.py:71-84 -- the reference runs the whole step as one VM
// function, llama_exec_graph.py:126).
//
// Each phase is the weight-streaming tcgen05 projection of linear_tc.cu (swap-AB, stream-K ranges over a
// persistent grid, TMEM double buffering, LoRA expand as extra MMA stages, TMA-store epilogue) with the same
// tile split, so results are bit-identical to the separate launches.  What the chain removes is the fixed
// cost between them:
//   * the weight producer never stops: weights and adapter B tiles are constants, so it streams the next
//     phase's first stages into the shared-memory ring while the grid is still finishing the current one;
//   * phases are separated by grid-wide barriers in global memory (one arrival per CTA, acquire spin by one
//     thread per waiting role) instead of kernel boundaries; only the token-tile producer waits for "input
//     rows complete", only the LoRA operand builder waits for "shrink outputs complete";
//   * the row operations between projections run inside the kernel on the output warps: residual add +
//     RMSNorm (one CTA per row, the reduction order of residual_rmsnorm_kernel) and the LoRA shrink (one warp
//     per (row, rank index), the order of lora_shrink_kernel), the latter off the critical path.
// All CTAs must be co-resident (grid <= SM count, one CTA per SM by shared memory).  Every wait -- mbarrier,
// split-tile counter, grid barrier -- is bounded; a CTA that gives up sets a bit in the status word, which
// makes every other wait of the grid return early, and the last CTA to leave resets the barrier counters.
#include <atomic>
#include <mutex>

#include "linear.cuh"
#include "tc_ptx.cuh"

namespace mlora {
namespace {

constexpr int BM = 128;
constexpr int kThreads = 224;  // warp 0 weight producer, 1 MMA issuer, 2..5 output warps, 6 token-tile producer
constexpr int kMaxPhases = MLORA_CHAIN_MAX_PHASES;
constexpr int kBarsPerPhase = 3;  // norm done, shrink done, projection done
constexpr int kMaxGrid = 256;
// scratch layout (shared with mlora_linear): status word at 0, exit ticket at 8, grid barriers from 64,
// split-tile tickets from 256, fp32 partial tiles behind them
constexpr int kHeaderBytes = 256;
constexpr int kExitOffset = 8;
constexpr int kBarOffset = 64;
static_assert(kBarOffset + kMaxPhases * kBarsPerPhase * 4 <= kHeaderBytes, "barriers must fit the header");

enum : int { kStWProducer = 1, kStMma = 2, kStEpilogue = 4, kStAcc = 8, kStXProducer = 16, kStBuilder = 32,
             kStCache = 64, kStPartials = 128, kStGridBarrier = 256 };

struct PhaseDev {
  // projection
  const uint8_t* W;   // pre-tiled weights (mlora_pack_weight)
  const uint8_t* Bp;  // pre-tiled adapter B stack (mlora_pack_lora_b) or nullptr
  const float* u;     // [T, n_mod*r_max] shrink outputs
  int in, out, k_blocks, row_tiles, per_cta;
  int flags;          // MLORA_SILU_MUL | MLORA_OUT_F32
  int r_max, n_mod;   // shrink: rank pitch per module and modules sharing the input (u rows hold n_mod*r_max)
  int e_nmod;         // expand: modules along the output rows (an interleaved gate/up stack counts as one of twice the pitch)
  int lora_sub, n_sub;
  int mod_off[5];
  int x_wait, u_wait, done_bar;  // barrier indices, -1 = none
  // residual add + RMSNorm in front of the projection (res == nullptr: none); writes the projection's input rows
  const bf16* delta;
  float* res;
  const bf16* norm_w;
  bf16* xn;
  float eps;
  int norm_wait, norm_done;
  // LoRA shrink in front of the projection (A == nullptr: none); reads the projection's input rows
  const bf16* A;
  const bf16* xin;
  int64_t ldx;
  float* u_out;
  int shrink_wait, shrink_done;
};

struct ChainParams {  // passed by value as the kernel's parameter block
  CUtensorMap map_x[kMaxPhases];
  CUtensorMap map_y[kMaxPhases];
  PhaseDev ph[kMaxPhases];
  int n_phases, T, n_adapters;
  const int32_t* slots;
  const int32_t* ranks;
  const float* scales;
  int32_t* status;
  int32_t* exit_ticket;
  int32_t* bars;
  int32_t* tickets;
  float* partials;
};

static_assert(sizeof(ChainParams) <= 4000, "the parameter block must fit the kernel parameter space");

template <int BN>
struct Cfg {
  static constexpr int kWBytes = BM * BK * 2;
  static constexpr int kXBytes = BN * BK * 2;
  static constexpr int kXStages = 8;  // token tiles come from L2: a shallow ring leaves the shared memory to the weight stream
  static constexpr int kCacheBytes = 16 * 1024;  // LoRA B operands (scaled, masked shrink outputs) of the token tile
  static constexpr int kOutBytes = 32 * BM * 4;  // staging of one 32-token output chunk
  static constexpr int kAuxBytes = 1024 + 5 * BN * 4 + kCacheBytes + kOutBytes;
  static constexpr int kBudget = 227 * 1024 - 1024 - 256;
  static constexpr int kWStages0 = (kBudget - kAuxBytes - kXStages * kXBytes) / kWBytes;
  static constexpr int kWStages = kWStages0 > 10 ? 10 : kWStages0;
  static constexpr int kSmemBytes = kWStages * kWBytes + kXStages * kXBytes + kAuxBytes + 1024;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kChunk = BN < 32 ? BN : 32;
};

struct Range {
  int it0, it1;
};
struct Segment {
  int tile, kb0, kb1;
};
__device__ __forceinline__ Range cta_range(const PhaseDev& p, int cta) {
  const long long total = (long long)p.row_tiles * p.k_blocks;
  long long a = (long long)cta * p.per_cta, b = a + p.per_cta;
  if (a > total) a = total;
  if (b > total) b = total;
  return Range{(int)a, (int)b};
}
__device__ __forceinline__ Segment next_segment(const PhaseDev& p, int& it, int it1) {
  Segment s;
  s.tile = it / p.k_blocks;
  s.kb0 = it - s.tile * p.k_blocks;
  s.kb1 = min(p.k_blocks, s.kb0 + (it1 - it));
  it += s.kb1 - s.kb0;
  return s;
}
__device__ __forceinline__ int module_of(const PhaseDev& p, int o) {
  int m = 0;
#pragma unroll 1
  while (m + 1 < p.e_nmod && o >= p.mod_off[m + 1]) ++m;
  return m;
}
template <int BN>
__device__ __forceinline__ bool lora_cached(const PhaseDev& p, int n_seg) {
  return n_seg * p.n_sub * BN * p.lora_sub * 2 <= Cfg<BN>::kCacheBytes;
}

// ---- grid-wide barriers ---------------------------------------------------------------------------------------
__device__ __forceinline__ void grid_arrive(int32_t* bar) {
  asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(bar) : "memory");
}
// One thread spins (bounded) until `target` CTAs have arrived; gives up early when this CTA or any other has
// recorded a failure.
__device__ __forceinline__ bool grid_wait(const int32_t* bar, int target, const int32_t* status, volatile int* abort) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    int seen;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(bar) : "memory");
    if (seen >= target) return true;
    if ((spin & 63) == 63) {
      int st;
      asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(status) : "memory");
      if (st != 0 || *abort) return false;
    }
    __nanosleep(40);
  }
  return false;
}
__device__ __forceinline__ void proxy_fence_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Distinct adapter slots among the T rows, in order of first appearance (one full warp).
template <int BN>
__device__ __forceinline__ int distinct_slots(const int32_t* slots, int T, int n_adapters, int* s_tok, int* s_list) {
  const int lane = threadIdx.x & 31;
  for (int n = lane; n < BN; n += 32) {
    int s = n < T ? slots[n] : -1;
    s_tok[n] = (s >= 0 && s < n_adapters) ? s : -1;
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

// ---- row operations on the output warps (128 threads, named barrier 1) --------------------------------------------
// Residual add + RMSNorm of row `row`: res += delta; xn = res * rsqrt(mean(res^2) + eps) * w.  The 128 threads stand
// in for the 256 threads of residual_rmsnorm_kernel, two each (e and e + 128), and reduce in that kernel's order, so
// the two produce the same bits.  H % 8 == 0, H <= 8192.
__device__ __forceinline__ void norm_row(const PhaseDev& p, int row, int etid, float* s_red /*[9]*/) {
  const int H = p.in;
  float* r = p.res + (size_t)row * H;
  const bf16* d = p.delta ? p.delta + (size_t)row * H : nullptr;
  const int lane = etid & 31, w = etid >> 5;
  float keep[2][4][8];
  float ss[2] = {0.f, 0.f};
#pragma unroll
  for (int v = 0; v < 2; ++v) {
    float4 ra[4], rb[4];
    uint4 rd[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int k = (c * 256 + v * 128 + etid) * 8;
      if (k < H) {
        ra[c] = __ldcg(reinterpret_cast<const float4*>(r + k));
        rb[c] = __ldcg(reinterpret_cast<const float4*>(r + k + 4));
        if (d) rd[c] = __ldcg(reinterpret_cast<const uint4*>(d + k));
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int k = (c * 256 + v * 128 + etid) * 8;
      float(&x)[8] = keep[v][c];
      if (k < H) {
        x[0] = ra[c].x, x[1] = ra[c].y, x[2] = ra[c].z, x[3] = ra[c].w;
        x[4] = rb[c].x, x[5] = rb[c].y, x[6] = rb[c].z, x[7] = rb[c].w;
        if (d) {
          float df[8];
          unpack8(rd[c], df);
#pragma unroll
          for (int i = 0; i < 8; ++i) x[i] += df[i];
          *reinterpret_cast<float4*>(r + k) = make_float4(x[0], x[1], x[2], x[3]);
          *reinterpret_cast<float4*>(r + k + 4) = make_float4(x[4], x[5], x[6], x[7]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss[v] = fmaf(x[i], x[i], ss[v]);
      }
    }
  }
  const float s0 = warp_sum(ss[0]), s1 = warp_sum(ss[1]);
  if (lane == 0) {
    s_red[w] = s0;      // warps 0..3 of the 256-thread kernel
    s_red[4 + w] = s1;  // warps 4..7
  }
  epi_bar_sync();
  float t = lane < 8 ? s_red[lane] : 0.f;
  t = warp_sum(t);
  epi_bar_sync();  // s_red may be rewritten by the next row
  const float inv = rsqrtf(t / (float)H + p.eps);
#pragma unroll
  for (int v = 0; v < 2; ++v) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int k = (c * 256 + v * 128 + etid) * 8;
      if (k < H) {
        float wf[8], o[8];
        unpack8(ld_cached(p.norm_w + k), wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = keep[v][c][i] * inv * wf[i];
        *reinterpret_cast<uint4*>(p.xn + (size_t)row * H + k) = pack8(o);
      }
    }
  }
}

// u[t, j] = A[slot[t], j, :] . x[t, :] for one (t, j), by one warp, in the order of lora_shrink_kernel.
__device__ __forceinline__ void shrink_item(const PhaseDev& p, const ChainParams& P, int t, int j, int lane) {
  const int r_tot = p.r_max * p.n_mod, in = p.in;
  const int slot = P.slots[t];
  float acc = 0.f;
  const int jm = j % p.r_max;
  if (slot >= 0 && slot < P.n_adapters && (jm < 16 || jm < P.ranks[slot])) {
    const bf16* a = p.A + ((size_t)slot * r_tot + j) * in;
    const bf16* xr = p.xin + (size_t)t * p.ldx;
    for (int k0 = lane * 8; k0 < in; k0 += 256 * 8) {
      uint4 av[8], xv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int k = k0 + c * 256;
        if (k < in) {
          av[c] = ld_cached(a + k);
          xv[c] = __ldcg(reinterpret_cast<const uint4*>(xr + k));  // written earlier in this launch: not through L1
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (k0 + c * 256 < in) {
          float af[8], xf[8];
          unpack8(av[c], af);
          unpack8(xv[c], xf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc = fmaf(af[i], xf[i], acc);
        }
      }
    }
    acc = warp_sum(acc);
  }
  if (lane == 0) p.u_out[(size_t)t * r_tot + j] = acc;
}

// Profiling build only (-DMLORA_CHAIN_TRACE): every CTA records nanosecond timestamps of its phase events, read
// back with mlora_chain_trace_dump().  The shipped library is built without it.
#ifdef MLORA_CHAIN_TRACE
constexpr int kTraceEvents = 24;  // per (CTA, phase)
__device__ unsigned long long g_trace[kMaxGrid * kMaxPhases * kTraceEvents];
__device__ __forceinline__ void trace(int cta, int ph, int ev) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  g_trace[((size_t)cta * kMaxPhases + ph) * kTraceEvents + ev] = t;
}
#define TRACE(ph, ev) trace(cta, ph, ev)
#else
#define TRACE(ph, ev) ((void)0)
#endif

template <int BN>
__global__ void __launch_bounds__(kThreads, 1) decode_chain_kernel(const __grid_constant__ ChainParams P) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* w_ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* x_ring = w_ring + C::kWStages * C::kWBytes;
  uint8_t* s_cache = x_ring + C::kXStages * C::kXBytes;
  uint8_t* s_out = s_cache + C::kCacheBytes;
  uint8_t* aux = s_out + C::kOutBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(aux);
  uint64_t* empty_bar = full_bar + C::kWStages;
  uint64_t* xfull_bar = empty_bar + C::kWStages;
  uint64_t* xempty_bar = xfull_bar + C::kXStages;
  uint64_t* acc_full = xempty_bar + C::kXStages;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* cache_full = acc_empty + 2;
  uint64_t* cache_empty = cache_full + 1;
  uint64_t* preload_bar = cache_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(preload_bar + 1);
  int* p_list = reinterpret_cast<int*>(aux + 1024);  // weight producer: distinct slots
  int* x_tok = p_list + BN;                           // operand builder: slot of each row
  int* x_list = x_tok + BN;                           //                  distinct slots
  float* x_scale = reinterpret_cast<float*>(x_list + BN);
  int* s_tmp = reinterpret_cast<int*>(x_scale + BN);
  __shared__ int s_abort;
  __shared__ int s_flag;
  __shared__ int s_nseg;
  __shared__ float s_red[9];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;

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
      mbar_init(&acc_empty[b], 4);
    }
    mbar_init(cache_full, 1);
    mbar_init(cache_empty, 1);
    mbar_init(preload_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int ph = 0; ph < P.n_phases; ++ph) {
      tma_prefetch_desc(&P.map_x[ph]);
      tma_prefetch_desc(&P.map_y[ph]);
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The next kernel in the stream may become resident from here on; this kernel's weight producer starts at
  // once (weights are constants), every other role first waits until the kernels before it have completed.
  pdl_launch_dependents();
  if (warp != 0) pdl_wait();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- weight producer (one thread): W stages of every phase back to back, plus the adapter B tiles --------
    if (lane == 0) {
      int n = 0, n_seg = 0;
      bool ok = true, got_preload = false;
      const uint64_t pol = l2_policy_evict_first();
      for (int ph = 0; ph < P.n_phases && ok; ++ph) {
        const PhaseDev& p = P.ph[ph];
        const Range rg = cta_range(p, cta);
        const uint32_t rb = p.lora_sub * 2;
        int it = rg.it0;
        while (it < rg.it1 && ok) {
          const Segment sg = next_segment(p, it, rg.it1);
          for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++n) {
            const int s = n % C::kWStages, round = n / C::kWStages;
            if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &s_abort)) {
              s_abort = 1;
              atomicOr(P.status, kStWProducer);
              ok = false;
              break;
            }
            mbar_expect_tx(&full_bar[s], C::kWBytes);
            bulk_load_hint(w_ring + s * C::kWBytes, p.W + ((size_t)sg.tile * p.k_blocks + kb) * C::kWBytes, C::kWBytes,
                           &full_bar[s], pol);
          }
          if (ok && p.Bp != nullptr && sg.kb0 == 0) {
            // the tile's first k-blocks are ours: this CTA also runs the tile's LoRA stages, after them
            if (!got_preload) {
              if (!mbar_wait(preload_bar, 0, &s_abort)) {
                s_abort = 1;
                atomicOr(P.status, kStWProducer);
                ok = false;
                break;
              }
              n_seg = s_nseg;
              got_preload = true;
            }
            const int n_l = n_seg * p.n_sub;
            const int group = lora_cached<BN>(p, n_seg) ? C::kWBytes / (BM * (int)rb) : 1;
            const int n_groups = (n_l + group - 1) / group;
            for (int g = 0; g < n_groups && ok; ++g, ++n) {
              const int s = n % C::kWStages, round = n / C::kWStages;
              if (!mbar_wait(&empty_bar[s], (round & 1) ^ 1, &s_abort)) {
                s_abort = 1;
                atomicOr(P.status, kStWProducer);
                ok = false;
                break;
              }
              const int l0 = g * group, l1 = min(n_l, l0 + group);
              mbar_expect_tx(&full_bar[s], (l1 - l0) * BM * rb);
              for (int l = l0; l < l1; ++l) {
                const int slot = p_list[l / p.n_sub], sb = l % p.n_sub;
                bulk_load_hint(w_ring + s * C::kWBytes + (l - l0) * BM * rb,
                               p.Bp + (((size_t)slot * p.row_tiles + sg.tile) * p.n_sub + sb) * (BM * rb), BM * rb,
                               &full_bar[s], pol);
              }
            }
          }
        }
      }
    }
  } else if (warp == 6) {
    // ---- token-tile producer: lane 0 issues the x copies; all lanes build the LoRA B operands ----------------
    int n = 0, n_seg = 0, cur_key = -1, n_build = 0;
    bool ok = true, got_preload = false;
    for (int ph = 0; ph < P.n_phases && ok; ++ph) {
      const PhaseDev& p = P.ph[ph];
      const Range rg = cta_range(p, cta);
      if (rg.it0 >= rg.it1) continue;
      const uint32_t rb = p.lora_sub * 2;
      const int r_tot = p.r_max * p.n_mod;
      if (p.x_wait >= 0) {  // the rows this phase reads are complete (all CTAs' stores, or the row operation)
        int w = 1;
        if (lane == 0) w = grid_wait(P.bars + p.x_wait, G, P.status, &s_abort) ? 1 : 0;
        w = __shfl_sync(0xffffffffu, w, 0);
        if (!w) {
          if (lane == 0) {
            s_abort = 1;
            atomicOr(P.status, kStGridBarrier);
          }
          ok = false;
          break;
        }
        proxy_fence_all();  // the acquire above orders generic accesses; the copies below go through the async proxy
      }
      if (lane == 0) TRACE(ph, 5);
      bool u_ready = p.u_wait < 0 || p.u_wait == p.x_wait;
      int it = rg.it0;
      while (it < rg.it1 && ok) {
        const Segment sg = next_segment(p, it, rg.it1);
        if (lane == 0) {
          int nn = n;
          for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++nn) {
            const int s = nn % C::kXStages, round = nn / C::kXStages;
            if (!mbar_wait(&xempty_bar[s], (round & 1) ^ 1, &s_abort)) {
              s_abort = 1;
              atomicOr(P.status, kStXProducer);
              ok = false;
              break;
            }
            mbar_expect_tx(&xfull_bar[s], C::kXBytes);
            tma_load_2d(x_ring + s * C::kXBytes, &P.map_x[ph], kb * BK, 0, &xfull_bar[s]);
          }
        }
        n += sg.kb1 - sg.kb0;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!(ok && p.Bp != nullptr && sg.kb0 == 0)) continue;
        if (!got_preload) {
          int w = 1;
          if (lane == 0) w = mbar_wait(preload_bar, 0, &s_abort) ? 1 : 0;
          w = __shfl_sync(0xffffffffu, w, 0);
          if (!w) {
            if (lane == 0) {
              s_abort = 1;
              atomicOr(P.status, kStBuilder);
            }
            ok = false;
            break;
          }
          n_seg = s_nseg;
          got_preload = true;
        }
        if (!u_ready) {  // the shrink outputs of this phase are complete
          int w = 1;
          if (lane == 0) w = grid_wait(P.bars + p.u_wait, G, P.status, &s_abort) ? 1 : 0;
          w = __shfl_sync(0xffffffffu, w, 0);
          if (!w) {
            if (lane == 0) {
              s_abort = 1;
              atomicOr(P.status, kStGridBarrier);
            }
            ok = false;
            break;
          }
          u_ready = true;
          if (lane == 0) TRACE(ph, 9);
        }
        // B operand of a LoRA stage = scale * u of the rows that use the adapter (zero rows for the others) in the
        // swizzled K-major layout the MMA expects: once per (phase, module) into the shared-memory cache when all
        // of them fit, else stage by stage into the token-tile ring.
        const int mod = module_of(p, sg.tile * BM);
        const int u_off = mod * p.r_max;
        const int chunks = p.lora_sub / 8;
        const bool cached = lora_cached<BN>(p, n_seg);
        const int key = ph * 8 + mod;
        if (cached && key == cur_key) continue;
        if (cached) {
          int w = 1;
          if (lane == 0) w = mbar_wait(cache_empty, (n_build & 1) ^ 1, &s_abort) ? 1 : 0;
          w = __shfl_sync(0xffffffffu, w, 0);
          if (!w) {
            if (lane == 0) {
              s_abort = 1;
              atomicOr(P.status, kStBuilder);
            }
            ok = false;
            break;
          }
          const int n_vec = n_seg * p.n_sub * BN * (int)rb / 16;
          for (int i = lane; i < n_vec; i += 32) reinterpret_cast<uint4*>(s_cache)[i] = make_uint4(0u, 0u, 0u, 0u);
          __syncwarp();
          const int per_row = chunks * p.n_sub;
          for (int idx = lane; idx < BN * per_row; idx += 32) {
            const int nrow = idx / per_row, rem = idx - nrow * per_row;
            const int sb = rem / chunks, c = rem - sb * chunks;
            const int slot = x_tok[nrow];
            if (slot < 0) continue;
            int sgi = 0;
            while (x_list[sgi] != slot) ++sgi;  // the slot is in the list by construction
            const float sc = x_scale[sgi];
            const float* ur = p.u + (size_t)nrow * r_tot + u_off + sb * p.lora_sub + c * 8;
            const float4 lo = __ldcg(reinterpret_cast<const float4*>(ur));
            const float4 hi = __ldcg(reinterpret_cast<const float4*>(ur + 4));
            const float f[8] = {lo.x * sc, lo.y * sc, lo.z * sc, lo.w * sc, hi.x * sc, hi.y * sc, hi.z * sc, hi.w * sc};
            const int sw = rb == 128 ? (nrow & 7) : rb == 64 ? ((nrow >> 1) & 3) : ((nrow >> 2) & 1);
            *reinterpret_cast<uint4*>(s_cache + (sgi * p.n_sub + sb) * BN * rb + nrow * rb + ((c ^ sw) << 4)) = pack8(f);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(cache_full);
          cur_key = key;
          ++n_build;
          continue;
        }
        for (int sgi = 0; sgi < n_seg && ok; ++sgi) {
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
                atomicOr(P.status, kStXProducer);
              }
              ok = false;
              break;
            }
            uint8_t* xt = x_ring + s * C::kXBytes;
            for (int idx = lane; idx < BN * chunks; idx += 32) {
              const int nrow = idx / chunks, c = idx - nrow * chunks;
              uint4 val = make_uint4(0u, 0u, 0u, 0u);
              if (x_tok[nrow] == slot) {
                const float* ur = p.u + (size_t)nrow * r_tot + u_off + sb * p.lora_sub + c * 8;
                const float4 lo = __ldcg(reinterpret_cast<const float4*>(ur));
                const float4 hi = __ldcg(reinterpret_cast<const float4*>(ur + 4));
                const float f[8] = {lo.x * sc, lo.y * sc, lo.z * sc, lo.w * sc, hi.x * sc, hi.y * sc, hi.z * sc, hi.w * sc};
                val = pack8(f);
              }
              const int sw = rb == 128 ? (nrow & 7) : rb == 64 ? ((nrow >> 1) & 3) : ((nrow >> 2) & 1);
              *reinterpret_cast<uint4*>(xt + nrow * rb + ((c ^ sw) << 4)) = val;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&xfull_bar[s]);
            ++n;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (one thread) ----------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      const uint32_t xfull0 = smem_u32(xfull_bar), xempty0 = smem_u32(xempty_bar);
      const uint64_t adesc0 = make_smem_desc(smem_u32(w_ring)), bdesc0 = make_smem_desc(smem_u32(x_ring));
      int nw = 0, nx = 0, j = 0, n_seg = 0, cur_key = -1, n_build = 0;
      bool ok = true, got_preload = false;
      for (int ph = 0; ph < P.n_phases && ok; ++ph) {
        const PhaseDev& p = P.ph[ph];
        const Range rg = cta_range(p, cta);
        const uint32_t rb = p.lora_sub * 2;
        int it = rg.it0;
        while (it < rg.it1 && ok) {
          const Segment sg = next_segment(p, it, rg.it1);
          const int buf = j & 1;
          const uint32_t d_tmem = tmem_base + buf * BN;
          int n_l = 0, group = 1;
          bool cached = false, new_build = false;
          if (p.Bp != nullptr && sg.kb0 == 0) {
            if (!got_preload) {
              if (!mbar_wait(preload_bar, 0, &s_abort)) {
                s_abort = 1;
                atomicOr(P.status, kStMma);
                ok = false;
                break;
              }
              n_seg = s_nseg;
              got_preload = true;
            }
            n_l = n_seg * p.n_sub;
            cached = lora_cached<BN>(p, n_seg);
            if (cached) {
              group = C::kWBytes / (BM * (int)rb);
              const int key = ph * 8 + module_of(p, sg.tile * BM);
              new_build = key != cur_key;
              cur_key = key;
            }
          }
          const int n_groups = (n_l + group - 1) / group;
          const int n_w = sg.kb1 - sg.kb0;
          if (!mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, &s_abort)) {
            s_abort = 1;
            atomicOr(P.status, kStAcc);
            ok = false;
            break;
          }
          tc_fence_after();
          {
            // The stream's inner loop, one thread: ring positions, parities, barrier addresses and descriptors are
            // kept in registers and advanced by additions (no division, no address conversion per stage).
            int ws = nw % C::kWStages, xs = nx % C::kXStages;
            uint32_t wpar = (nw / C::kWStages) & 1, xpar = (nx / C::kXStages) & 1;
            for (int l = 0; l < n_w && ok; ++l) {
              if (!mbar_wait_a(full0 + 8 * ws, wpar, &s_abort) || !mbar_wait_a(xfull0 + 8 * xs, xpar, &s_abort)) {
                s_abort = 1;
                atomicOr(P.status, kStMma);
                ok = false;
                break;
              }
              tc_fence_after();
#ifdef MLORA_CHAIN_TRACE
              if (it - (sg.kb1 - sg.kb0) == rg.it0 && l == 0) TRACE(ph, 12);  // first stage of the phase consumed
              if (it >= rg.it1 && l == n_w - 1) TRACE(ph, 13);                // last stage of the phase consumed
              if (it - (sg.kb1 - sg.kb0) == rg.it0 && l == 12) TRACE(ph, 14); // 13th stage
#endif
              const uint64_t adesc = adesc0 + (uint64_t)(ws * (C::kWBytes >> 4));  // start-address field, 16-byte units
              const uint64_t bdesc = bdesc0 + (uint64_t)(xs * (C::kXBytes >> 4));
              umma_bf16(d_tmem, adesc, bdesc, idesc, l > 0 ? 1u : 0u);
#pragma unroll
              for (int k = 1; k < BK / 16; ++k) umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
              umma_commit_a(empty0 + 8 * ws);
              umma_commit_a(xempty0 + 8 * xs);
              if (++ws == C::kWStages) {
                ws = 0;
                wpar ^= 1;
              }
              if (++xs == C::kXStages) {
                xs = 0;
                xpar ^= 1;
              }
              ++nw;
              ++nx;
            }
          }
          if (cached && new_build && ok) {
            // every MMA that read the previous cache contents has been issued: the builder may overwrite them
            // once those MMAs retire; then wait for the new contents
            if (n_build > 0) umma_commit(cache_empty);
            if (!mbar_wait(cache_full, n_build & 1, &s_abort)) {
              s_abort = 1;
              atomicOr(P.status, kStCache);
              ok = false;
            }
            tc_fence_after();
            ++n_build;
          }
          for (int g = 0; g < n_groups && ok; ++g, ++nw) {
            const int s = nw % C::kWStages;
            int xs = 0;
            bool got = mbar_wait(&full_bar[s], (nw / C::kWStages) & 1, &s_abort);
            if (got && !cached) {
              xs = nx % C::kXStages;
              got = mbar_wait(&xfull_bar[xs], (nx / C::kXStages) & 1, &s_abort);
            }
            if (!got) {
              s_abort = 1;
              atomicOr(P.status, kStMma);
              ok = false;
              break;
            }
            tc_fence_after();
            const int l0 = g * group, l1 = min(n_l, l0 + group);
            for (int l = l0; l < l1; ++l) {
              const uint64_t adesc = make_smem_desc(smem_u32(w_ring + s * C::kWBytes + (l - l0) * BM * rb), rb);
              const uint64_t bdesc =
                  make_smem_desc(cached ? smem_u32(s_cache + l * BN * rb) : smem_u32(x_ring + xs * C::kXBytes), rb);
              for (int k = 0; k < p.lora_sub / 16; ++k) umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
            }
            umma_commit(&empty_bar[s]);
            if (!cached) {
              umma_commit(&xempty_bar[xs]);
              ++nx;
            }
          }
          if (ok) umma_commit(&acc_full[buf]);
          ++j;
        }
      }
    }
  } else {
    // ---- output warps 2..5: row operations, then the epilogue of each phase ------------------------------------------
    const int q = warp & 3;
    const int etid = q * 32 + lane;  // 0..127 = row inside the tile; TMEM lane quarter = warp % 4
    int j = 0;
    bool ok = true;
    // per-row adapter slots, distinct list and scales: the same for every phase of the chain
    if (q == 0) {
      const int ns = P.slots ? distinct_slots<BN>(P.slots, P.T, P.n_adapters, x_tok, s_tmp) : 0;
      for (int i = lane; i < ns; i += 32) {
        p_list[i] = x_list[i] = s_tmp[i];
        x_scale[i] = P.scales ? P.scales[s_tmp[i]] : 0.f;
      }
      if (lane == 0) s_nseg = ns;
      __syncwarp();
      if (lane == 0) mbar_arrive(preload_bar);
    }

    auto wait_grid = [&](int bar) -> bool {  // all 128 threads
      if (etid == 0) {
        const bool got = grid_wait(P.bars + bar, G, P.status, &s_abort);
        s_flag = got ? 1 : 0;
        if (!got) {
          s_abort = 1;
          atomicOr(P.status, kStGridBarrier);
        }
      }
      epi_bar_sync();
      const bool got = s_flag != 0;
      epi_bar_sync();
      return got;
    };
    auto arrive_grid = [&](int bar) {  // all 128 threads; their global writes are ordered before the arrival
      __threadfence();
      proxy_fence_all();
      epi_bar_sync();
      if (etid == 0) grid_arrive(P.bars + bar);
    };

    for (int ph = 0; ph < P.n_phases; ++ph) {
      const PhaseDev& p = P.ph[ph];
      if (etid == 0) TRACE(ph, 0);
      // ---- row operations in front of the projection --------------------------------------------------------
      if (p.res != nullptr) {
        if (ok && p.norm_wait >= 0) ok = wait_grid(p.norm_wait);
        if (etid == 0) TRACE(ph, 1);
        if (ok)
          for (int row = cta; row < P.T; row += G) norm_row(p, row, etid, s_red);
        arrive_grid(p.norm_done);
        if (etid == 0) TRACE(ph, 2);
      }
      if (p.A != nullptr) {
        if (ok && p.shrink_wait >= 0) ok = wait_grid(p.shrink_wait);
        if (etid == 0) TRACE(ph, 3);
        if (ok) {
          const int r_tot = p.r_max * p.n_mod, items = P.T * r_tot;
          for (int item = cta * 4 + q; item < items; item += G * 4) shrink_item(p, P, item / r_tot, item % r_tot, lane);
        }
        arrive_grid(p.shrink_done);
        if (etid == 0) TRACE(ph, 4);
      }
      // ---- epilogue of this CTA's segments ---------------------------------------------------------------------
      const Range rg = cta_range(p, cta);
      const bool silu = (p.flags & MLORA_SILU_MUL) != 0;
      const bool out_f32 = (p.flags & MLORA_OUT_F32) != 0;
      int it = rg.it0;
      while (it < rg.it1 && ok) {
        const Segment sg = next_segment(p, it, rg.it1);
        const int buf = j & 1;
        const bool full_seg = sg.kb0 == 0 && sg.kb1 == p.k_blocks;

        // v[i] = (token c0+i, output row etid of the tile): SiLU*up, staging, one TMA store (which clips tokens >= T
        // and outputs >= out)
        auto finish = [&](float(&v)[32], int c0) {
          if (etid == 0) bulk_wait_read0();  // the previous chunk's store has finished reading s_out
          if (etid == 0) TRACE(ph, 16);
          epi_bar_sync();
          if (etid == 0) TRACE(ph, 17);
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
          if (etid == 0) TRACE(ph, 18);
          epi_bar_sync();
          if (etid == 0) tma_store_2d(&P.map_y[ph], s_out, silu ? sg.tile * (BM / 2) : sg.tile * BM, c0);
          if (etid == 0) TRACE(ph, 19);
        };

        // Split tile: contributors = the CTAs whose ranges meet the tile's k-blocks; the one holding its FIRST
        // k-blocks (it reaches them at the end of its range) finishes the tile.
        long long ts = 0, te = 0;
        int c_first = 0, c_last = 0;
        if (!full_seg) {
          ts = (long long)sg.tile * p.k_blocks;
          te = ts + p.k_blocks;
          c_first = (int)(ts / p.per_cta);
          c_last = (int)((te - 1) / p.per_cta);
        }
        const bool finisher = !full_seg && cta == c_first;
        float pre[32];
        bool pre_have = true;
        if constexpr (BN <= 32) {
          if (finisher) {
            // collect the other contributors' partial sums now, while this CTA's own last MMAs still run
            if (etid == 0) {
              TRACE(ph, 20);
              const int need = c_last - c_first;
              bool got = false;
              for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
                int seen;
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(P.tickets + c_first) : "memory");
                if (seen >= need) {
                  got = true;
                  break;
                }
                if ((spin & 63) == 63) {  // a failure here or anywhere in the grid: the partials may never come
                  int st;
                  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(P.status) : "memory");
                  if (st != 0 || s_abort) break;
                }
                __nanosleep(64);
              }
              P.tickets[c_first] = 0;  // ready for the next phase / call
              s_flag = got ? 1 : 0;
              if (!got) {
                s_abort = 1;
                atomicOr(P.status, kStPartials);
              }
            }
            epi_bar_sync();
            if (etid == 0) TRACE(ph, 21);
            pre_have = s_flag != 0;
#pragma unroll
            for (int i = 0; i < C::kChunk; ++i) pre[i] = 0.f;
            if (pre_have) {
              for (int cc = c_first + 1; cc <= c_last; ++cc) {  // CTA order: deterministic
                const float* ps = P.partials + ((size_t)cc * 2) * (size_t)(BN * BM);
#pragma unroll
                for (int i = 0; i < C::kChunk; ++i) pre[i] += __ldcg(ps + (size_t)i * BM + etid);
              }
            }
            epi_bar_sync();  // s_flag is reused
            if (etid == 0) TRACE(ph, 22);
          }
        }

        if (!mbar_wait(&acc_full[buf], (j >> 1) & 1, &s_abort)) {
          if (!s_abort) {
            s_abort = 1;
            atomicOr(P.status, kStEpilogue);
          }
          ok = false;
          break;
        }
        tc_fence_after();
        if (etid == 0) TRACE(ph, it >= rg.it1 ? 7 : 6);
        const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
        float v[32];
        if (BN >= 32) tmem_ld32(t_addr, v); else tmem_ld16(t_addr, v);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);  // accumulator read: hand it back to the MMA warp
        if (etid == 0) TRACE(ph, 23);
        if (full_seg) {
          finish(v, 0);
        } else if (!finisher) {
          // slot 0 if this CTA's range starts inside the tile (always, except for c_first); kept general
          const bool starts_here = rg.it0 >= ts;
          float* part = P.partials + ((size_t)cta * 2 + (starts_here ? 0 : 1)) * (size_t)(BN * BM);
#pragma unroll
          for (int i = 0; i < C::kChunk; ++i) part[(size_t)i * BM + etid] = v[i];
          __threadfence();
          epi_bar_sync();
          if (etid == 0) atomicAdd(&P.tickets[c_first], 1);
        } else if (pre_have) {
#pragma unroll
          for (int i = 0; i < C::kChunk; ++i) v[i] += pre[i];
          finish(v, 0);
        } else {
          ok = false;
        }
        ++j;
      }
      // ---- this CTA's part of the phase is in global memory: tell the grid ---------------------------------------
      if (etid == 0) TRACE(ph, 8);
      if (p.done_bar >= 0) {
        if (etid == 0) bulk_wait_all0();  // the TMA stores have completed, not only read their source
        if (etid == 0) TRACE(ph, 10);
        arrive_grid(p.done_bar);
        if (etid == 0) TRACE(ph, 11);
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------------------------------------------
  if (warp == 4 && lane == 0) bulk_wait_all0();  // output thread 0 (warp 4, lane 0) issued the stores
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);  // copies that may still be in flight get time to land
  }
  if (warp == 1) tmem_dealloc(tmem_base, C::kTmemCols);
  if (tid == 0) {
    // the last CTA to leave puts the grid barriers (and, after a failure, the split-tile counters) back to zero
    __threadfence();
    const int old = atomicAdd(P.exit_ticket, 1);
    if (old == G - 1) {
      for (int i = 0; i < kMaxPhases * kBarsPerPhase; ++i) P.bars[i] = 0;
      int st;
      asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(P.status) : "memory");
      if (st != 0)
        for (int i = 0; i < kMaxGrid; ++i) P.tickets[i] = 0;
      __threadfence();
      *P.exit_ticket = 0;
    }
  }
}

int pick_bn(int T) { return T <= 16 ? 16 : 32; }

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
    return v > kMaxGrid ? kMaxGrid : v;
  }();
  return n;
}

template <int BN>
int launch(ChainParams& P, const mlora_chain_phase* ph, cudaStream_t st) {
  using C = Cfg<BN>;
  for (int i = 0; i < P.n_phases; ++i) {
    int rc = make_map(&P.map_x[i], ph[i].d_x, P.T, ph[i].in, ph[i].ldx, BN);
    if (rc) return rc;
    const bool f32 = (ph[i].flags & MLORA_OUT_F32) != 0, silu = (ph[i].flags & MLORA_SILU_MUL) != 0;
    rc = make_out_map(&P.map_y[i], ph[i].d_y, P.T, silu ? ph[i].out / 2 : ph[i].out, ph[i].ldy, BN < 32 ? BN : 32,
                      silu ? BM / 2 : BM, f32);
    if (rc) return rc;
  }
  static std::atomic<unsigned long long> attr_done{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!((attr_done.load(std::memory_order_acquire) >> (dev & 63)) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return fail(MLORA_ECUDA, "decode_chain: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  launch_pdl_if(pdl_enabled_gemm(), decode_chain_kernel<BN>, sm_count(), kThreads, C::kSmemBytes, st, P);
  count_launch();
  MLORA_CHECK_LAUNCH("decode_chain_kernel");
  return MLORA_OK;
}

}  // namespace
}  // namespace mlora

using namespace mlora;

#ifdef MLORA_CHAIN_TRACE
extern "C" int mlora_chain_trace_dump(void* host_buf, size_t bytes) {
  const size_t n = sizeof(unsigned long long) * kMaxGrid * kMaxPhases * kTraceEvents;
  return cudaMemcpyFromSymbol(host_buf, g_trace, bytes < n ? bytes : n) == cudaSuccess ? 0 : -2;
}
#endif

extern "C" int mlora_decode_chain(const mlora_chain_phase* phases, int32_t n_phases, int32_t T, const int32_t* d_slots,
                                  const int32_t* d_ranks, const float* d_scales, int32_t n_adapters, void* d_work,
                                  size_t work_bytes, void* stream) {
  MLORA_REQUIRE(phases && n_phases >= 1 && n_phases <= kMaxPhases, "decode_chain: 1..%d phases (got %d)", kMaxPhases, n_phases);
  MLORA_REQUIRE(T >= 0 && T <= 32, "decode_chain: decode-size batches only, T <= 32 (got %d)", T);
  MLORA_REQUIRE(d_work && aligned16(d_work), "decode_chain: a scratch buffer is required");
  if (T == 0) return MLORA_OK;
  const int bn = pick_bn(T);
  size_t need = 0;
  static ChainParams P;  // (too large for the stack of some callers' threads; filled and copied by the launch below)
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  P.n_phases = n_phases;
  P.T = T;
  P.n_adapters = n_adapters;
  P.slots = d_slots;
  P.ranks = d_ranks;
  P.scales = d_scales;
  const int G = sm_count();
  for (int i = 0; i < n_phases; ++i) {
    const mlora_chain_phase& h = phases[i];
    PhaseDev& p = P.ph[i];
    MLORA_REQUIRE(h.d_x && h.d_Wp && h.d_y, "decode_chain: phase %d: null pointer", i);
    MLORA_REQUIRE(h.in > 0 && h.out > 0 && h.in % 8 == 0 && h.ldx % 8 == 0, "decode_chain: phase %d: bad sizes in=%d out=%d", i, h.in, h.out);
    MLORA_REQUIRE(aligned16(h.d_x) && aligned16(h.d_Wp) && aligned16(h.d_y), "decode_chain: phase %d: 16-byte alignment", i);
    const bool f32 = (h.flags & MLORA_OUT_F32) != 0, silu = (h.flags & MLORA_SILU_MUL) != 0;
    MLORA_REQUIRE((h.flags & ~(MLORA_OUT_F32 | MLORA_SILU_MUL)) == 0, "decode_chain: phase %d: only OUT_F32 / SILU_MUL flags", i);
    MLORA_REQUIRE(!(f32 && silu), "decode_chain: phase %d: OUT_F32 with SILU_MUL", i);
    if (silu) MLORA_REQUIRE(h.out % 16 == 0, "decode_chain: phase %d: SILU_MUL needs out %% 16 == 0", i);
    const int es = f32 ? 4 : 2, cols = silu ? h.out / 2 : h.out;
    MLORA_REQUIRE((h.ldy * es) % 16 == 0 && (cols * es) % 16 == 0, "decode_chain: phase %d: output rows must be 16-byte multiples", i);
    p.W = (const uint8_t*)h.d_Wp;
    p.in = h.in;
    p.out = h.out;
    p.flags = h.flags;
    p.k_blocks = (h.in + BK - 1) / BK;
    p.row_tiles = (h.out + BM - 1) / BM;
    // the split of mlora_linear: equal contiguous ranges, at least 4 k-blocks per CTA
    const long long total = (long long)p.row_tiles * p.k_blocks;
    MLORA_REQUIRE(total < 2000000000ll, "decode_chain: phase %d too large", i);
    long long grid = G;
    if (grid > (total + 3) / 4) grid = (total + 3) / 4;
    if (grid < 1) grid = 1;
    p.per_cta = (int)((total + grid - 1) / grid);
    const size_t w = linear_tc_workspace(T, h.in, h.out);
    need = w > need ? w : need;
    // LoRA
    p.Bp = nullptr;
    p.u = nullptr;
    p.A = nullptr;
    p.r_max = 16;
    p.n_mod = 1;
    p.e_nmod = 1;
    p.lora_sub = 16;
    p.n_sub = 1;
    p.mod_off[0] = 0;
    p.mod_off[1] = h.out;
    p.u_wait = -1;
    p.shrink_wait = p.shrink_done = -1;
    const int prev_done = i > 0 ? (i - 1) * kBarsPerPhase + 2 : -1;
    // residual + RMSNorm in front
    p.res = nullptr;
    p.norm_wait = p.norm_done = -1;
    if (h.d_res) {
      MLORA_REQUIRE(h.d_norm_w && aligned16(h.d_res) && aligned16(h.d_norm_w) && (!h.d_delta || aligned16(h.d_delta)),
                    "decode_chain: phase %d: norm operands", i);
      MLORA_REQUIRE(h.in <= 8192 && h.ldx == h.in, "decode_chain: phase %d: the fused RMSNorm needs in <= 8192 and dense input rows", i);
      p.delta = (const bf16*)h.d_delta;
      p.res = h.d_res;
      p.norm_w = (const bf16*)h.d_norm_w;
      p.xn = (bf16*)const_cast<void*>(h.d_x);
      p.eps = h.eps;
      p.norm_wait = prev_done;
      p.norm_done = i * kBarsPerPhase + 0;
    }
    p.x_wait = h.d_res ? p.norm_done : prev_done;
    if (h.d_Bp) {
      MLORA_REQUIRE(h.d_A_all && h.d_u && d_slots && d_ranks && d_scales && n_adapters > 0, "decode_chain: phase %d: LoRA operands missing", i);
      MLORA_REQUIRE(aligned16(h.d_A_all) && aligned16(h.d_u) && aligned16(h.d_Bp), "decode_chain: phase %d: LoRA alignment", i);
      int r_max = h.r_max, n_mod = h.n_mod;
      MLORA_REQUIRE(n_mod >= 1 && n_mod <= 4, "decode_chain: phase %d: n_mod %d", i, n_mod);
      p.A = (const bf16*)h.d_A_all;
      p.xin = (const bf16*)h.d_x;
      p.ldx = h.ldx;
      p.u_out = h.d_u;
      p.shrink_wait = p.x_wait;
      p.shrink_done = i * kBarsPerPhase + 1;
      p.u_wait = p.shrink_done;
      p.u = h.d_u;
      p.Bp = (const uint8_t*)h.d_Bp;
      // the shrink works on (r_max, n_mod) as given; the expand sees an interleaved gate/up stack as one module
      // of twice the pitch (see mlora_linear)
      int e_rmax = r_max, e_nmod = n_mod;
      if (silu) {
        MLORA_REQUIRE(n_mod == 2, "decode_chain: phase %d: SILU_MUL implies n_mod == 2", i);
        e_rmax = 2 * r_max;
        e_nmod = 1;
      }
      MLORA_REQUIRE(e_rmax == 16 || e_rmax == 32 || e_rmax == 64 || e_rmax == 128, "decode_chain: phase %d: rank pitch %d", i, e_rmax);
      p.r_max = r_max;
      p.n_mod = n_mod;
      p.e_nmod = e_nmod;
      p.lora_sub = e_rmax < 64 ? e_rmax : 64;
      p.n_sub = e_rmax / p.lora_sub;
      if (e_nmod > 1)
        for (int m = 0; m <= e_nmod; ++m) p.mod_off[m] = h.mod_offsets[m];
      if (e_nmod > 1) {
        MLORA_REQUIRE(h.mod_offsets[0] == 0 && h.mod_offsets[n_mod] == h.out, "decode_chain: phase %d: module offsets must span [0,out]", i);
        for (int m = 1; m < n_mod; ++m) MLORA_REQUIRE(h.mod_offsets[m] % BM == 0, "decode_chain: phase %d: modules must be tile aligned", i);
      }
    }
    p.done_bar = i + 1 < n_phases ? i * kBarsPerPhase + 2 : -1;
  }
  if (work_bytes < need) return fail(MLORA_ESIZE, "decode_chain: workspace of %zu bytes needed, %zu given", need, work_bytes);
  P.status = (int32_t*)d_work;
  P.exit_ticket = (int32_t*)((uint8_t*)d_work + kExitOffset);
  P.bars = (int32_t*)((uint8_t*)d_work + kBarOffset);
  P.tickets = (int32_t*)((uint8_t*)d_work + kHeaderBytes);
  P.partials = (float*)((uint8_t*)d_work + kHeaderBytes + kMaxGrid * 4);
  return bn == 16 ? launch<16>(P, phases, (cudaStream_t)stream) : launch<32>(P, phases, (cudaStream_t)stream);
}
