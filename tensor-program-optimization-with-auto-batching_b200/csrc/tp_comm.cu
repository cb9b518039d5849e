// Tensor-parallel exchange over peer memory: the all-reduce that follows a row-parallel projection (o, down),
// fused with the residual add + RMSNorm that consumes it, as ONE kernel per rank that stores into and reads
// from the other GPUs' memory over NVLink -- no collective library call, no second pass over the data.
//
// One process per GPU.  Every rank owns an arena (cudaMalloc'ed here, exported as a CUDA IPC handle, mapped by
// the peers):  header | flags [2][8][T_max] | gather flags [2][T_max] | inbox [2][8][T_max * H] bf16 | gather box
// [2][T_max * H] bf16.
// One exchange, on rank r, CTA t (= row t of the [T, H] partial result):
//   1. push: row t of the local partial is stored into inbox[buf][r][t] of every peer (128-bit stores over
//      NVLink), fenced at system scope, then flags[buf][r][t] of every peer is set to the exchange number;
//   2. wait (bounded) until the own flags[buf][g][t] of every peer g carry that number: their row t has landed in
//      THIS GPU's memory (remote data is always read locally, never pulled across the link by a consumer);
//   3. sum the G rows in rank order in fp32 (the own one from registers) -- every rank computes the same bits --,
//      add the residual, RMSNorm, write.
// With more than four ranks the exchange is two-step instead (each rank would otherwise store its whole partial result
// seven times over): row t has an owner, rank t mod G; every rank stores its row t into the owner's inbox only, the owner
// sums the G rows in rank order, rounds the sum to bf16 and stores it into every peer's gather box (+ flag); the others
// wait for that one row.  Bytes out per rank: 2 (G-1)/G of the partial result instead of G-1 times it; same bits.
// Rows are independent, so no rank waits for more than the row it is about to use.  `buf` alternates with the
// exchange number: a rank can be at most one exchange ahead of a peer (it needs the peer's rows to finish one),
// so two buffers are enough.  The exchange number lives in the arena and is advanced by the last CTA of each
// launch, which keeps a launch replayable inside a CUDA graph.  No multicast load, no library kernel on peer
// memory; every wait is bounded and ends in a status bit, never in a hang.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace mlora {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kTpThreads = 256;
constexpr int kTpHeader = 256;  // int32: [0] exchange number, [1] exit ticket, [2] status
constexpr uint32_t kTpSpinDefault = 1u << 22;

struct TpCtx {
  int rank, world, T_max, H;
  size_t bytes;
  uint8_t* local;
  uint8_t* peer[kMaxWorld];
  bool open[kMaxWorld];
  uint32_t spin_limit;
  int two_step;
};

struct TpArgs {
  uint8_t* local;
  uint8_t* peer[kMaxWorld];
  int rank, world, T_max, H, T;
  const bf16* partial;  // [T, H] this rank's partial sums
  float* res;           // [T, H] residual in/out, or nullptr: plain all-reduce
  const bf16* w;        // [H] norm weight
  float eps;
  bf16* out;            // [T, H]: RMSNorm(res) * w, or the plain sum
  uint32_t spin_limit;
  int two_step;         // rows have owners (rank t mod world): reduce there, gather the rounded sums
};

__host__ __device__ inline size_t flags_off(int T_max, int buf, int src, int t) {
  return kTpHeader + ((size_t)(buf * kMaxWorld + src) * T_max + t) * sizeof(int32_t);
}
__host__ __device__ inline size_t gflags_off(int T_max, int buf, int t) {
  return kTpHeader + (size_t)2 * kMaxWorld * T_max * sizeof(int32_t) + ((size_t)buf * T_max + t) * sizeof(int32_t);
}
__host__ __device__ inline size_t inbox_base(int T_max) {
  size_t b = kTpHeader + (size_t)2 * (kMaxWorld + 1) * T_max * sizeof(int32_t);
  return (b + 255) & ~(size_t)255;
}
__host__ __device__ inline size_t inbox_off(int T_max, int H, int buf, int src, int t) {
  return inbox_base(T_max) + (((size_t)(buf * kMaxWorld + src) * T_max + t) * H) * sizeof(bf16);
}
__host__ __device__ inline size_t gbox_off(int T_max, int H, int buf, int t) {
  return inbox_base(T_max) + ((size_t)2 * kMaxWorld * T_max * H + ((size_t)buf * T_max + t) * H) * sizeof(bf16);
}
size_t arena_bytes(int T_max, int H) { return gbox_off(T_max, H, 1, T_max); }

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float block_sum256(float v, float* sm /*[33]*/) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sm[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < kTpThreads / 32 ? sm[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) sm[32] = t;
  }
  __syncthreads();
  const float r = sm[32];
  __syncthreads();
  return r;
}

// NCH chunks of 8 elements per thread: H <= 2048 * NCH.
template <int NCH>
__global__ void __launch_bounds__(kTpThreads) tp_allreduce_norm_kernel(TpArgs a) {
  __shared__ int s_epoch;
  __shared__ int s_ok;
  __shared__ float sm[33];
  const int t = blockIdx.x, tid = threadIdx.x;
  int32_t* hdr = reinterpret_cast<int32_t*>(a.local);
  if (tid == 0) {
    s_epoch = hdr[0] + 1;  // written by the last CTA of the previous exchange on this stream
    s_ok = 1;
  }
  __syncthreads();
  const int epoch = s_epoch, buf = epoch & 1;
  const int H = a.H;

  // ---- 1. push this rank's row to every peer ----------------------------------------------------------------------
  uint4 mine[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = (c * kTpThreads + tid) * 8;
    if (k < H) mine[c] = *reinterpret_cast<const uint4*>(a.partial + (size_t)t * H + k);
  }
  const bool two = a.two_step != 0;
  const int owner = two ? t % a.world : a.rank;  // (one-step: every rank reduces every row itself)
  const bool reduce_here = owner == a.rank;
  for (int g = 0; g < a.world; ++g) {
    if (g == a.rank || (two && g != owner)) continue;
    bf16* dst = reinterpret_cast<bf16*>(a.peer[g] + inbox_off(a.T_max, H, buf, a.rank, t));
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int k = (c * kTpThreads + tid) * 8;
      if (k < H) *reinterpret_cast<uint4*>(dst + k) = mine[c];
    }
  }
  // The CTA barrier orders every thread's stores before the flag stores below, whose system-scope release makes them
  // (cumulatively) visible to whoever acquires the flag: the row is in the peer's memory before its flag says so.
  __syncthreads();
  if (tid < a.world && tid != a.rank && (!two || tid == owner))
    st_release_sys(reinterpret_cast<int32_t*>(a.peer[tid] + flags_off(a.T_max, buf, a.rank, t)), epoch);

  // ---- 2. wait for row t of every peer (it lands in this GPU's own memory) -------------------------------------------
  if (reduce_here && tid < a.world && tid != a.rank) {
    const int32_t* f = reinterpret_cast<const int32_t*>(a.local + flags_off(a.T_max, buf, tid, t));
    bool got = false;
    for (uint32_t spin = 0; spin < a.spin_limit; ++spin) {
      if (ld_acquire_sys(f) >= epoch) {
        got = true;
        break;
      }
      __nanosleep(100);
    }
    if (!got) {
      s_ok = 0;
      atomicOr(&hdr[2], 1 << tid);  // which peer's row never came
    }
  }
  // two-step, row owned elsewhere: wait for the owner's rounded sum instead
  if (!reduce_here && tid == 0) {
    const int32_t* f = reinterpret_cast<const int32_t*>(a.local + gflags_off(a.T_max, buf, t));
    bool got = false;
    for (uint32_t spin = 0; spin < a.spin_limit; ++spin) {
      if (ld_acquire_sys(f) >= epoch) {
        got = true;
        break;
      }
      __nanosleep(100);
    }
    if (!got) {
      s_ok = 0;
      atomicOr(&hdr[2], 1 << owner);
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;

  // ---- 3. sum in rank order (rounded to bf16: the value a separate all-reduce would have delivered), or take the
  //         owner's; then residual, RMSNorm ------------------------------------------------------------------------------
  uint4 total[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = (c * kTpThreads + tid) * 8;
    total[c] = make_uint4(0u, 0u, 0u, 0u);
    if (k >= H) continue;
    if (reduce_here) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int g = 0; g < a.world; ++g) {
        uint4 raw = mine[c];
        if (g != a.rank) {
          raw = make_uint4(0u, 0u, 0u, 0u);
          if (ok) raw = __ldcg(reinterpret_cast<const uint4*>(a.local + inbox_off(a.T_max, H, buf, g, t)) + (k >> 3));
        }
        float f[8];
        unpack8(raw, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      total[c] = pack8(acc);
    } else if (ok) {
      total[c] = __ldcg(reinterpret_cast<const uint4*>(a.local + gbox_off(a.T_max, H, buf, t)) + (k >> 3));
    }
  }
  if (two && reduce_here) {  // (uniform per CTA) hand the rounded sum to every peer
    for (int g = 0; g < a.world; ++g) {
      if (g == a.rank) continue;
      bf16* dst = reinterpret_cast<bf16*>(a.peer[g] + gbox_off(a.T_max, H, buf, t));
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int k = (c * kTpThreads + tid) * 8;
        if (k < H) *reinterpret_cast<uint4*>(dst + k) = total[c];
      }
    }
    __syncthreads();
    if (tid < a.world && tid != a.rank)
      st_release_sys(reinterpret_cast<int32_t*>(a.peer[tid] + gflags_off(a.T_max, buf, t)), epoch);
  }
  float v[NCH][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = (c * kTpThreads + tid) * 8;
    if (k < H) {
      if (a.res) {
        float acc[8];
        unpack8(total[c], acc);
        float* r = a.res + (size_t)t * H + k;
        const float4 r0 = *reinterpret_cast<const float4*>(r), r1 = *reinterpret_cast<const float4*>(r + 4);
        v[c][0] = r0.x + acc[0], v[c][1] = r0.y + acc[1], v[c][2] = r0.z + acc[2], v[c][3] = r0.w + acc[3];
        v[c][4] = r1.x + acc[4], v[c][5] = r1.y + acc[5], v[c][6] = r1.z + acc[6], v[c][7] = r1.w + acc[7];
        *reinterpret_cast<float4*>(r) = make_float4(v[c][0], v[c][1], v[c][2], v[c][3]);
        *reinterpret_cast<float4*>(r + 4) = make_float4(v[c][4], v[c][5], v[c][6], v[c][7]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[c][i], v[c][i], ss);
      } else {
        *reinterpret_cast<uint4*>(a.out + (size_t)t * H + k) = total[c];
      }
    }
  }
  if (a.res) {
    ss = block_sum256(ss, sm);
    const float inv = rsqrtf(ss / (float)H + a.eps);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int k = (c * kTpThreads + tid) * 8;
      if (k < H) {
        float wf[8], o[8];
        unpack8(ld_cached(a.w + k), wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = v[c][i] * inv * wf[i];
        *reinterpret_cast<uint4*>(a.out + (size_t)t * H + k) = pack8(o);
      }
    }
  }

  // ---- 4. the last CTA to leave advances the exchange number ----------------------------------------------------------------
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const int old = atomicAdd(&hdr[1], 1);
    if (old == (int)gridDim.x - 1) {
      hdr[1] = 0;
      hdr[0] = epoch;
      __threadfence();
    }
  }
}

}  // namespace
}  // namespace mlora

using namespace mlora;

extern "C" size_t mlora_tp_arena_bytes(int32_t T_max, int32_t H) {
  if (T_max <= 0 || H <= 0) return 0;
  return arena_bytes(T_max, H);
}

extern "C" int mlora_tp_create(int32_t rank, int32_t world, int32_t T_max, int32_t H, void** ctx_out) {
  MLORA_REQUIRE(ctx_out, "tp_create: null pointer");
  MLORA_REQUIRE(world >= 1 && world <= kMaxWorld && rank >= 0 && rank < world, "tp_create: rank %d of %d (at most %d ranks)", rank,
                world, kMaxWorld);
  MLORA_REQUIRE(T_max > 0 && H > 0 && H % 8 == 0 && H <= 2048 * 4, "tp_create: T_max=%d, H=%d (H a multiple of 8 up to 8192)", T_max, H);
  TpCtx* c = new TpCtx();
  c->rank = rank;
  c->world = world;
  c->T_max = T_max;
  c->H = H;
  c->bytes = arena_bytes(T_max, H);
  c->spin_limit = kTpSpinDefault;
  c->two_step = world > 4;  // measured: the one-step push wins at 2 and 4 ranks, loses to NCCL at 8
  if (const char* e = getenv("MLORA_TP_TWO_STEP")) c->two_step = e[0] == '1';
  for (int g = 0; g < kMaxWorld; ++g) {
    c->peer[g] = nullptr;
    c->open[g] = false;
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, c->bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, c->bytes);
  if (e != cudaSuccess) {
    delete c;
    return fail(MLORA_ECUDA, "tp_create: %s", cudaGetErrorString(e));
  }
  c->local = (uint8_t*)p;
  c->peer[rank] = c->local;
  *ctx_out = c;
  return MLORA_OK;
}

extern "C" int mlora_tp_export(void* ctx, void* handle_out64) {
  MLORA_REQUIRE(ctx && handle_out64, "tp_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ((TpCtx*)ctx)->local);
  if (e != cudaSuccess) return fail(MLORA_ECUDA, "tp_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  memcpy(handle_out64, &h, 64);
  return MLORA_OK;
}

extern "C" int mlora_tp_connect(void* ctx, int32_t peer_rank, const void* handle64) {
  MLORA_REQUIRE(ctx && handle64, "tp_connect: null pointer");
  TpCtx* c = (TpCtx*)ctx;
  MLORA_REQUIRE(peer_rank >= 0 && peer_rank < c->world && peer_rank != c->rank, "tp_connect: bad peer rank %d", peer_rank);
  MLORA_REQUIRE(!c->open[peer_rank], "tp_connect: peer %d is connected already", peer_rank);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(MLORA_ECUDA, "tp_connect: cudaIpcOpenMemHandle(peer %d): %s", peer_rank, cudaGetErrorString(e));
  c->peer[peer_rank] = (uint8_t*)p;
  c->open[peer_rank] = true;
  return MLORA_OK;
}

extern "C" int mlora_tp_set_spin_limit(void* ctx, uint32_t polls) {
  MLORA_REQUIRE(ctx && polls > 0, "tp_set_spin_limit: bad arguments");
  ((TpCtx*)ctx)->spin_limit = polls;
  return MLORA_OK;
}

// Status word of this rank's arena (bit g set: a row of rank g never arrived) -- synchronises the device.
extern "C" int mlora_tp_status(void* ctx, int32_t* status_out) {
  MLORA_REQUIRE(ctx && status_out, "tp_status: null pointer");
  TpCtx* c = (TpCtx*)ctx;
  cudaError_t e = cudaMemcpy(status_out, c->local + 2 * sizeof(int32_t), sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(MLORA_ECUDA, "tp_status: %s", cudaGetErrorString(e));
  return MLORA_OK;
}

// Back to exchange number 0 with clean flags: every rank calls it, between two host-side barriers, after an
// exchange has failed (the ranks' exchange numbers may then disagree).
extern "C" int mlora_tp_reset(void* ctx) {
  MLORA_REQUIRE(ctx, "tp_reset: null pointer");
  TpCtx* c = (TpCtx*)ctx;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemset(c->local, 0, inbox_base(c->T_max));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(MLORA_ECUDA, "tp_reset: %s", cudaGetErrorString(e));
  return MLORA_OK;
}

extern "C" int mlora_tp_destroy(void* ctx) {
  MLORA_REQUIRE(ctx, "tp_destroy: null pointer");
  TpCtx* c = (TpCtx*)ctx;
  for (int g = 0; g < c->world; ++g)
    if (c->open[g]) cudaIpcCloseMemHandle(c->peer[g]);
  cudaFree(c->local);
  delete c;
  return MLORA_OK;
}

extern "C" int mlora_tp_allreduce_rmsnorm(void* ctx, const void* d_partial, float* d_res, const void* d_w, float eps,
                                          void* d_out, int32_t T, int32_t H, void* stream) {
  MLORA_REQUIRE(ctx, "tp_allreduce_rmsnorm: null context");
  TpCtx* c = (TpCtx*)ctx;
  MLORA_REQUIRE(T >= 0 && T <= c->T_max && H == c->H, "tp_allreduce_rmsnorm: T=%d H=%d, the arena was made for T <= %d, H = %d", T, H,
                c->T_max, c->H);
  // one CTA per row, and CTAs of different GPUs wait for one another: all of a launch's CTAs must be resident at once
  MLORA_REQUIRE(T <= 512, "tp_allreduce_rmsnorm: at most 512 rows per exchange (got %d)", T);
  MLORA_REQUIRE(d_partial && d_out && aligned16(d_partial) && aligned16(d_out), "tp_allreduce_rmsnorm: partial / out pointers");
  if (d_res) MLORA_REQUIRE(d_w && aligned16(d_res) && aligned16(d_w), "tp_allreduce_rmsnorm: residual / weight pointers");
  for (int g = 0; g < c->world; ++g)
    MLORA_REQUIRE(c->peer[g] != nullptr, "tp_allreduce_rmsnorm: peer %d is not connected", g);
  if (T == 0) return MLORA_OK;
  TpArgs a;
  a.local = c->local;
  for (int g = 0; g < kMaxWorld; ++g) a.peer[g] = g < c->world ? c->peer[g] : nullptr;
  a.rank = c->rank;
  a.world = c->world;
  a.T_max = c->T_max;
  a.H = H;
  a.T = T;
  a.partial = (const bf16*)d_partial;
  a.res = d_res;
  a.w = (const bf16*)d_w;
  a.eps = eps;
  a.out = (bf16*)d_out;
  a.spin_limit = c->spin_limit;
  a.two_step = c->world > 1 ? c->two_step : 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (H <= 2048)
    tp_allreduce_norm_kernel<1><<<T, kTpThreads, 0, st>>>(a);
  else if (H <= 4096)
    tp_allreduce_norm_kernel<2><<<T, kTpThreads, 0, st>>>(a);
  else if (H <= 6144)
    tp_allreduce_norm_kernel<3><<<T, kTpThreads, 0, st>>>(a);
  else
    tp_allreduce_norm_kernel<4><<<T, kTpThreads, 0, st>>>(a);
  count_launch();
  MLORA_CHECK_LAUNCH("tp_allreduce_norm_kernel");
  return MLORA_OK;
}
