// LSTM forward recurrence as ONE cooperative kernel for the whole sequence (bf16, B <= 128, H = 8 * G with
// G <= number of SMs; the translation stages use H = 1024: 128 CTAs).
//
// CTA c owns hidden units u0 = 8c .. 8c+7, i.e. the 32 gate columns {g*H + u0 + j}.  Its slice of W_hh
// (32 x H, 64 KB at H = 1024) is loaded into shared memory once and stays there for all T steps.  Per step:
// the previous hidden state h_{t-1} ([B, H], a slab of the output y) streams through a ring of TMA stages,
// tcgen05.mma accumulates the [128 x 32] recurrent projection in tensor memory, and the epilogue warps - one
// thread per batch row, which then holds all four gates of its 8 units - add the input projection and the
// bias, apply the cell update (cell state kept in registers across steps) and write h_t, c_t and the gate
// activations.  A grid-wide counter separates the steps: a CTA starts loading h_t only when all CTAs have
// published their part of it.  Compared with one contraction launch plus one cell launch per step this
// removes the launches, the round trip of the projection through HBM and the per-step reload of W_hh.
//
// Every wait is bounded; a wait that runs out (or an error seen by another role / CTA) sets the error word
// of the tensor-core kernels and makes every role leave its loop, after which tensor memory is freed.
#include "pd_gemm.cuh"
#include "pd_sm100_ptx.cuh"
#include <mutex>

namespace {

using namespace pd_sm100;

constexpr int kThreads = 192;            // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: cell epilogue
constexpr int kUnits = 8;                // hidden units per CTA
constexpr int kCols = 4 * kUnits;        // gate columns per CTA = MMA N
constexpr uint32_t kStageBytes = 128 * kBlockK * 2;      // one [128 x 64] K-block of h: 16 KiB
constexpr uint32_t kWBlockBytes = kCols * kBlockK * 2;   // one [32 x 64] K-block of the W_hh slice: 4 KiB

struct LstmP {
  int T, B, H, G, num_stages;
  int Bt, b0;                  // the tensors hold Bt batch rows per time step; this launch works on rows b0 .. b0 + B - 1
  uint32_t stage_bytes;        // one K-block of the h tile in shared memory: 128 rows (16 KiB), or 64 rows when B <= 64
  const __nv_bfloat16* gx;     // [T, B, 4H]
  const __nv_bfloat16* b_hh;   // [4H] or null
  __nv_bfloat16* y;            // [T, B, H]
  __nv_bfloat16* act;          // [T, B, 4H]
  float* c_all;                // [T, B, H]
  unsigned int* counter;       // zeroed before the launch
  int* err;
  uint32_t idesc;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One thread waits for the grid-wide counter; returns false when the bound ran out or an error is pending.  The poll
// is the link of the per-step chain that every CTA sits on: it is one acquire load per trip, and the error word
// (another round trip to L2) and the clock are looked at on every 32nd trip only.
__device__ __forceinline__ bool wait_counter(const unsigned int* counter, unsigned int target, int* err, int code) {
  const long long t0 = clock64();
  unsigned int trips = 0;
  while (ld_acquire(counter) < target) {
    if ((++trips & 31u) == 0u) {
      if (*(volatile int*)err != 0) return false;
      if (clock64() - t0 > kWaitCycles) { atomicCAS(err, 0, code); return false; }
    }
  }
  return true;
}

// Publish after a named barrier of the 128 epilogue threads: their global writes are ordered before the barrier,
// one thread then makes them visible device-wide and counts this CTA in (the pattern of a cooperative grid sync).
__device__ __forceinline__ void publish_step(unsigned int* counter, bool elected) {
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (elected) {
    __threadfence();
    atomicAdd(counter, 1u);
  }
}

// mbarrier wait that also gives up when another role or CTA has reported an error
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*(volatile int*)err != 0) return false;
    if (clock64() - t0 > kWaitCycles) {
      atomicCAS(err, 0, code);
      return false;
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 t = __bfloat1622float2(p[k]);
    f[2 * k] = t.x;
    f[2 * k + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) p[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return u;
}

__global__ void __launch_bounds__(kThreads, 1)
lstm_fwd_persistent_kernel(const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_w,
                           const LstmP p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[8];
  __shared__ __align__(8) uint64_t empty_bar[8];
  __shared__ __align__(8) uint64_t w_bar;
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_holder;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = p.num_stages;
  const int kblocks = p.H / kBlockK;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_w = smem0;                                        // kblocks x 4 KiB
  const uint32_t smem_a = smem0 + (uint32_t)kblocks * kWBlockBytes;     // S x 16 KiB (a multiple of 1024 in)
  const int u0 = blockIdx.x * kUnits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&w_bar), 1);
    mbar_init(smem_u32(&acc_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_holder)), "r"(32u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_base_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      // the W_hh slice: per K-block four boxes of 8 rows (one per gate), 8 rows = one swizzle atom
      mbar_expect_tx(smem_u32(&w_bar), (uint32_t)kblocks * kWBlockBytes);
      for (int kb = 0; kb < kblocks; ++kb)
        for (int g = 0; g < 4; ++g)
          tma_load_2d(smem_w + (uint32_t)kb * kWBlockBytes + (uint32_t)g * 1024u, &map_w, smem_u32(&w_bar), kb * kBlockK,
                      g * p.H + u0);
      uint32_t it = 0;
      bool ok = true;
      for (int t = 1; t < p.T && ok; ++t) {
        // every CTA has published its part of h_{t-1}
        const unsigned int target = (unsigned int)p.G * (unsigned int)t;
        ok = wait_counter(p.counter, target, p.err, 5);
        if (!ok) break;
        asm volatile("fence.proxy.async;" ::: "memory");      // the TMA reads below come after what was just observed
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = (int)(it % (uint32_t)S);
          const uint32_t ph = (it / (uint32_t)S) & 1u;
          if (!wait_bar(smem_u32(&empty_bar[s]), ph ^ 1u, p.err, 1)) { ok = false; break; }
          const uint32_t fb = smem_u32(&full_bar[s]);
          mbar_expect_tx(fb, p.stage_bytes);
          tma_load_2d(smem_a + (uint32_t)s * p.stage_bytes, &map_h, fb, kb * kBlockK, (t - 1) * p.Bt + p.b0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      bool ok = wait_bar(smem_u32(&w_bar), 0, p.err, 6);
      // The issuing thread runs every instruction between two MMAs itself and an N = 32 MMA is only 16 cycles of
      // tensor-pipe work, so descriptors advance by 32-bit adds on their low words and the ring position is
      // carried along instead of being derived by division.
      const uint64_t da0 = make_desc(smem_a, 0), db0 = make_desc(smem_w, 0);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
      const uint32_t idesc = p.idesc;
      int s = 0;
      uint32_t ph = 0, a_lo = a_lo0, fb = full0, eb = empty0;
      for (int t = 1; t < p.T && ok; ++t) {
        uint32_t b_lo = b_lo0;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!wait_bar(fb, ph, p.err, 2)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (kb == 0) umma_lo<1, 0>(tmem_acc, a_lo, a_hi, b_lo, b_hi, idesc, 0u);
          else umma_lo<1, 1>(tmem_acc, a_lo, a_hi, b_lo, b_hi, idesc, 1u);
#pragma unroll
          for (int kk = 1; kk < kBlockK / 16; ++kk)
            umma_lo<1, 1>(tmem_acc, a_lo + kk * 2, a_hi, b_lo + kk * 2, b_hi, idesc, 1u);
          umma_commit(eb);
          b_lo += kWBlockBytes >> 4;
          ++s; a_lo += p.stage_bytes >> 4; fb += 8; eb += 8;
          if (s == S) { s = 0; ph ^= 1u; a_lo = a_lo0; fb = full0; eb = empty0; }
        }
        if (ok) umma_commit(smem_u32(&acc_bar));
      }
    }
  } else {
    // ------------------------------ cell epilogue ------------------------------
    const int lg = warp & 3;                       // TMEM lane group of this warp
    const int b = lg * 32 + lane;                  // batch row
    const bool row = b < p.B;
    const int H = p.H;
    float c[kUnits];
#pragma unroll
    for (int j = 0; j < kUnits; ++j) c[j] = 0.f;
    float bias[kCols];
#pragma unroll
    for (int g = 0; g < 4; ++g)
#pragma unroll
      for (int j = 0; j < kUnits; ++j)
        bias[g * kUnits + j] = p.b_hh != nullptr ? __bfloat162float(p.b_hh[g * H + u0 + j]) : 0.f;
    bool ok = true;
    for (int t = 0; t < p.T && ok; ++t) {
      // input projection of this row: four 16-byte pieces (one per gate), in flight while the MMAs run
      uint4 gxv[4];
      const int64_t row4 = ((int64_t)t * p.Bt + p.b0 + (row ? b : 0)) * 4 * H + u0;
#pragma unroll
      for (int g = 0; g < 4; ++g) gxv[g] = *reinterpret_cast<const uint4*>(p.gx + row4 + (int64_t)g * H);
      uint32_t r[kCols];
      uint4 hold[4];                                 // gate activations of this step, stored after the publish
      if (t > 0) {
        ok = wait_bar(smem_u32(&acc_bar), (uint32_t)(t - 1) & 1u, p.err, 3);
        // one decision for all four epilogue warps (they meet at a named barrier further down)
        unsigned int all_ok;
        asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.and.pred p, 2, 128, q;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(all_ok) : "r"((unsigned int)ok) : "memory");
        ok = all_ok != 0;
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_ld32(tmem_acc + ((uint32_t)(lg * 32) << 16), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < kCols; ++j) r[j] = 0u;
      }
      if (row) {
        float pre[kCols];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float f[8];
          unpack8(gxv[g], f);
#pragma unroll
          for (int j = 0; j < kUnits; ++j) {
            float v = f[j];
            if (t > 0) v += __uint_as_float(r[g * kUnits + j]);
            if (p.b_hh != nullptr) v += bias[g * kUnits + j];
            pre[g * kUnits + j] = v;
          }
        }
        float hi[kUnits], ai[kUnits], af[kUnits], ag[kUnits], ao[kUnits];
#pragma unroll
        for (int j = 0; j < kUnits; ++j) {
          ai[j] = sigmoidf_(pre[j]);
          af[j] = sigmoidf_(pre[kUnits + j]);
          ag[j] = tanhf(pre[2 * kUnits + j]);
          ao[j] = sigmoidf_(pre[3 * kUnits + j]);
          c[j] = af[j] * c[j] + ai[j] * ag[j];
          hi[j] = ao[j] * tanhf(c[j]);
        }
        const int64_t rowh = ((int64_t)t * p.Bt + p.b0 + b) * H + u0;
        *reinterpret_cast<uint4*>(p.y + rowh) = pack8(hi);
        hold[0] = pack8(ai); hold[1] = pack8(af); hold[2] = pack8(ag); hold[3] = pack8(ao);
      }
      // publish: the accumulator has been read (the next step may overwrite it) and h_t is written
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      publish_step(p.counter, warp == 2 && lane == 0);
      // what only the backward pass reads goes out after the other CTAs have been let go
      if (row) {
        const int64_t rowh = ((int64_t)t * p.Bt + p.b0 + b) * H + u0;
        float4* cp = reinterpret_cast<float4*>(p.c_all + rowh);
        cp[0] = make_float4(c[0], c[1], c[2], c[3]);
        cp[1] = make_float4(c[4], c[5], c[6], c[7]);
        __nv_bfloat16* ap = p.act + ((int64_t)t * p.Bt + p.b0 + b) * 4 * H + u0;
        *reinterpret_cast<uint4*>(ap) = hold[0];
        *reinterpret_cast<uint4*>(ap + H) = hold[1];
        *reinterpret_cast<uint4*>(ap + 2 * (int64_t)H) = hold[2];
        *reinterpret_cast<uint4*>(ap + 3 * (int64_t)H) = hold[3];
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(32u) : "memory");
  }
}


// ------------------------------------------------------------------------------------------------
// Backward recurrence, whole sequence in one cooperative kernel (bf16, B <= 128, H a power of two in
// 128..1024: G = (H/128)^2 CTAs).  Two phases per step, separated by a grid-wide counter:
//   A(t): cell backward.  CTA c owns the U = H/G hidden units from c*U for all rows: dh = dy[t] + dh_acc,
//         dgates[t] from the saved activations and cell states, dc carried in a scratch array, dh_acc cleared.
//   B(t): dh_acc += dgates[t] . W_hh.  CTA (ns, ks) contracts the K slice [512 ks, 512 ks + 512) of the 4H gate
//         columns into the 128 units of slice ns: its [512 x 128] piece of W_hh sits in shared memory for the
//         whole sequence (MN-major operand, read in place), dgates[t] streams in by TMA, 32 MMAs of
//         128 x 128 x 16 accumulate in tensor memory and the epilogue adds the tile to dh_acc with red.v4.f32.
// ------------------------------------------------------------------------------------------------
constexpr int kBwdStages = 4;
constexpr int kBwdN = 128;               // units per N slice
constexpr int kBwdK = 512;               // gate columns per K slice
constexpr uint32_t kBwdWBytes = kBwdK * kBwdN * 2;       // 128 KiB

struct LstmBwdP {
  int T, B, H, G, U, NS;
  int Bt, b0;                   // as in LstmP
  const __nv_bfloat16* dy;      // [T, B, H]
  const __nv_bfloat16* act;     // [T, B, 4H]
  const float* c_all;           // [T, B, H]
  __nv_bfloat16* dgates;        // [T, B, 4H]
  float* dh_acc;                // [B, H], zeroed before the launch
  float* dc;                    // [B, H], zeroed before the launch
  unsigned int* counter;        // zeroed before the launch
  int* err;
  uint32_t idesc;
};


// AND of a flag over the 128 epilogue threads (named barrier 2)
__device__ __forceinline__ bool all_epilogue(bool ok) {
  unsigned int r;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.and.pred p, 2, 128, q;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(r) : "r"((unsigned int)ok) : "memory");
  return r != 0;
}

__global__ void __launch_bounds__(kThreads, 1)
lstm_bwd_persistent_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_w,
                           const LstmBwdP p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kBwdStages];
  __shared__ __align__(8) uint64_t empty_bar[kBwdStages];
  __shared__ __align__(8) uint64_t w_bar;
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_holder;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_w = smem0;                       // 8 K-blocks x 2 atoms x 8 KiB
  const uint32_t smem_a = smem0 + kBwdWBytes;          // kBwdStages x 16 KiB
  const int ns = blockIdx.x % p.NS, ks = blockIdx.x / p.NS;
  constexpr int kKb = kBwdK / kBlockK;                 // 8 K-blocks per step

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&w_bar), 1);
    mbar_init(smem_u32(&acc_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_holder)), "r"(128u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_acc = tmem_base_holder;

  // step index i = T-1-t; arrivals: after A_i the counter reaches G*(2i+1), after B_i G*(2i+2)
  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(smem_u32(&w_bar), kBwdWBytes);
      for (int kb = 0; kb < kKb; ++kb)
        for (int j = 0; j < 2; ++j)
          tma_load_2d(smem_w + (uint32_t)(kb * 2 + j) * kAtomBytes, &map_w, smem_u32(&w_bar), ns * kBwdN + j * 64,
                      ks * kBwdK + kb * kBlockK);
      uint32_t it = 0;
      bool ok = true;
      for (int i = 0; i + 1 < p.T && ok; ++i) {
        const int t = p.T - 1 - i;
        if (!wait_counter(p.counter, (unsigned int)p.G * (unsigned int)(2 * i + 1), p.err, 5)) break;
        asm volatile("fence.proxy.async;" ::: "memory");
        for (int kb = 0; kb < kKb; ++kb, ++it) {
          const int s = (int)(it % (uint32_t)kBwdStages);
          const uint32_t ph = (it / (uint32_t)kBwdStages) & 1u;
          if (!wait_bar(smem_u32(&empty_bar[s]), ph ^ 1u, p.err, 1)) { ok = false; break; }
          const uint32_t fb = smem_u32(&full_bar[s]);
          mbar_expect_tx(fb, kStageBytes);
          tma_load_2d(smem_a + (uint32_t)s * kStageBytes, &map_g, fb, ks * kBwdK + kb * kBlockK, t * p.Bt + p.b0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = wait_bar(smem_u32(&w_bar), 0, p.err, 6);
      // lean issue loop: see the forward kernel
      const uint64_t da0 = make_desc(smem_a, 0), db0 = make_desc(smem_w, 1);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
      const uint32_t idesc = p.idesc;
      int s = 0;
      uint32_t ph = 0, a_lo = a_lo0, fb = full0, eb = empty0;
      for (int i = 0; i + 1 < p.T && ok; ++i) {
        uint32_t b_lo = b_lo0;
        for (int kb = 0; kb < kKb; ++kb) {
          if (!wait_bar(fb, ph, p.err, 2)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (kb == 0) umma_lo<1, 0>(tmem_acc, a_lo, a_hi, b_lo, b_hi, idesc, 0u);
          else umma_lo<1, 1>(tmem_acc, a_lo, a_hi, b_lo, b_hi, idesc, 1u);
#pragma unroll
          for (int kk = 1; kk < kBlockK / 16; ++kk)
            umma_lo<1, 1>(tmem_acc, a_lo + kk * 2, a_hi, b_lo + kk * 128, b_hi, idesc, 1u);
          umma_commit(eb);
          b_lo += (2u * kAtomBytes) >> 4;
          ++s; a_lo += kStageBytes >> 4; fb += 8; eb += 8;
          if (s == kBwdStages) { s = 0; ph ^= 1u; a_lo = a_lo0; fb = full0; eb = empty0; }
        }
        if (ok) umma_commit(smem_u32(&acc_bar));
      }
    }
  } else {
    const int lg = warp & 3;
    const int b = lg * 32 + lane;
    const bool row = b < p.B;
    const int H = p.H;
    const int ua = blockIdx.x * p.U;               // first unit of this CTA's phase-A slice
    bool ok = true;
    for (int i = 0; i < p.T && ok; ++i) {
      const int t = p.T - 1 - i;
      // ---- phase A(t): needs every CTA's B(t+1) contribution to dh_acc
      if (i > 0) {
        bool mine = true;
        if (warp == 2 && lane == 0) mine = wait_counter(p.counter, (unsigned int)p.G * (unsigned int)(2 * i), p.err, 7);
        ok = all_epilogue(mine);
        if (!ok) break;
      }
      if (row) {
        for (int u = ua; u < ua + p.U; u += 8) {
          const int64_t e = ((int64_t)t * p.Bt + p.b0 + b) * H + u;         // [T,Bt,H] element
          const int64_t e4 = ((int64_t)t * p.Bt + p.b0 + b) * 4 * H + u;    // [T,Bt,4H] element of gate 0
          const int64_t bh = (int64_t)b * H + u;
          float dyf[8], ai[8], af[8], ag[8], ao[8];
          unpack8(*reinterpret_cast<const uint4*>(p.dy + e), dyf);
          unpack8(*reinterpret_cast<const uint4*>(p.act + e4), ai);
          unpack8(*reinterpret_cast<const uint4*>(p.act + e4 + H), af);
          unpack8(*reinterpret_cast<const uint4*>(p.act + e4 + 2 * (int64_t)H), ag);
          unpack8(*reinterpret_cast<const uint4*>(p.act + e4 + 3 * (int64_t)H), ao);
          const float4 h0 = __ldcg(reinterpret_cast<const float4*>(p.dh_acc + bh));
          const float4 h1 = __ldcg(reinterpret_cast<const float4*>(p.dh_acc + bh) + 1);
          const float4 d0 = *reinterpret_cast<const float4*>(p.dc + bh);
          const float4 d1 = *(reinterpret_cast<const float4*>(p.dc + bh) + 1);
          const float4 c0 = *reinterpret_cast<const float4*>(p.c_all + e);
          const float4 c1 = *(reinterpret_cast<const float4*>(p.c_all + e) + 1);
          float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0;
          if (t > 0) {
            q0 = *reinterpret_cast<const float4*>(p.c_all + e - (int64_t)p.Bt * H);
            q1 = *(reinterpret_cast<const float4*>(p.c_all + e - (int64_t)p.Bt * H) + 1);
          }
          const float dhv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
          const float dcv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
          const float ct[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
          const float cp[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
          float gi[8], gf[8], gg[8], go[8], dcn[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float dh = dyf[j] + dhv[j];
            const float tc = tanhf(ct[j]);
            const float dcj = dh * ao[j] * (1.f - tc * tc) + dcv[j];
            const float d_o = dh * tc;
            dcn[j] = dcj * af[j];
            gi[j] = dcj * ag[j] * ai[j] * (1.f - ai[j]);
            gf[j] = dcj * cp[j] * af[j] * (1.f - af[j]);
            gg[j] = dcj * ai[j] * (1.f - ag[j] * ag[j]);
            go[j] = d_o * ao[j] * (1.f - ao[j]);
          }
          __nv_bfloat16* gp = p.dgates + e4;
          *reinterpret_cast<uint4*>(gp) = pack8(gi);
          *reinterpret_cast<uint4*>(gp + H) = pack8(gf);
          *reinterpret_cast<uint4*>(gp + 2 * (int64_t)H) = pack8(gg);
          *reinterpret_cast<uint4*>(gp + 3 * (int64_t)H) = pack8(go);
          float4* dcp = reinterpret_cast<float4*>(p.dc + bh);
          dcp[0] = make_float4(dcn[0], dcn[1], dcn[2], dcn[3]);
          dcp[1] = make_float4(dcn[4], dcn[5], dcn[6], dcn[7]);
          float4* dhp = reinterpret_cast<float4*>(p.dh_acc + bh);
          dhp[0] = make_float4(0.f, 0.f, 0.f, 0.f);
          dhp[1] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      publish_step(p.counter, warp == 2 && lane == 0);
      if (t == 0) break;
      // ---- phase B(t): add this CTA's tile of dgates[t] . W_hh to dh_acc
      ok = all_epilogue(wait_bar(smem_u32(&acc_bar), (uint32_t)i & 1u, p.err, 3));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int cc = 0; cc < kBwdN; cc += 32) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_acc + ((uint32_t)(lg * 32) << 16) + (uint32_t)cc, r);
        tmem_ld_wait();
        if (row) {
          float* o = p.dh_acc + (int64_t)b * H + ns * kBwdN + cc;
#pragma unroll
          for (int q = 0; q < 8; ++q)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                         ::"l"(o + q * 4), "f"(__uint_as_float(r[q * 4])), "f"(__uint_as_float(r[q * 4 + 1])),
                           "f"(__uint_as_float(r[q * 4 + 2])), "f"(__uint_as_float(r[q * 4 + 3]))
                         : "memory");
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      publish_step(p.counter, warp == 2 && lane == 0);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(128u) : "memory");
  }
}

int g_bwd_state[64];

// Grid-barrier counters of the backward kernel: a ring of slots, one per call (a cooperative kernel owns the
// whole GPU while it runs, so far fewer than 64 calls are ever in flight on one device).
__device__ unsigned int g_bwd_counters[64];
unsigned int* g_bwd_counter_base[64];
unsigned int g_bwd_next[64];

std::mutex g_mu;
int g_state[64];          // per device: 0 unknown, 1 usable, -1 not usable

}  // namespace

// Returns PD_OK when the sequence was enqueued, 1 when this path does not apply (the caller then runs the
// per-step path), or an error code.  `counter` must point at 4 bytes of device scratch.
int pd_lstm_fwd_persistent(const void* gx, const void* w_hh, const void* b_hh, int T, int B, int H, void* y, void* act,
                           float* c_all, unsigned int* counter, cudaStream_t s) {
  return pd_lstm_fwd_persistent_rows(gx, w_hh, b_hh, T, B, 0, B, H, y, act, c_all, counter, s);
}

// The same on the batch rows b0 .. b0 + B - 1 of tensors that hold Bt rows per time step.  Two such launches on two
// streams (the halves of a batch) run side by side: with B <= 64 the h tile is staged 64 rows at a time and a CTA
// takes half of an SM's shared memory, so both grids are resident at once and each hides the other's waits.
int pd_lstm_fwd_persistent_rows(const void* gx, const void* w_hh, const void* b_hh, int T, int Bt, int b0, int B, int H,
                                void* y, void* act, float* c_all, unsigned int* counter, cudaStream_t s) {
  if (B > 128 || H % kBlockK != 0 || H % kUnits != 0 || T < 2 || b0 < 0 || b0 + B > Bt) return 1;
  const int G = H / kUnits;
  const int kblocks = H / kBlockK;
  const uint32_t w_bytes = (uint32_t)kblocks * kWBlockBytes;
  if (w_bytes > 96u * 1024u) return 1;
  const bool half = B <= 64 && B < Bt;       // one of several launches that share the GPU
  const uint32_t stage_bytes = half ? kStageBytes / 2 : kStageBytes;
  const uint32_t budget = half ? 96u * 1024u : 200u * 1024u;     // half: two CTAs (105 KiB each with the slack) per SM
  if (w_bytes + 2 * stage_bytes > budget) return 1;
  int stages = (int)((budget - w_bytes) / stage_bytes);
  if (stages > 8) stages = 8;
  if (stages < 2) return 1;
  // (an MMA reads 128 rows from a stage's start: with 64-row stages the last one needs 8 KiB of slack behind it)
  const size_t smem = (size_t)w_bytes + (size_t)stages * stage_bytes + (half ? kStageBytes / 2 : 0) + 1024;
  int dev = 0;
  PD_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return 1;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_state[dev] == 0) {
      int coop = 0, per_sm = 0;
      PD_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
      PD_CUDA(cudaFuncSetAttribute(lstm_fwd_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
      PD_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lstm_fwd_persistent_kernel, kThreads, 200 * 1024));
      g_state[dev] = (coop && per_sm >= 1) ? 1 : -1;
    }
    if (g_state[dev] < 0) return 1;
  }
  if (G > pd_num_sms()) return 1;

  LstmP p;
  memset(&p, 0, sizeof(p));
  p.T = T; p.B = B; p.H = H; p.G = G; p.num_stages = stages;
  p.Bt = Bt; p.b0 = b0; p.stage_bytes = stage_bytes;
  p.gx = (const __nv_bfloat16*)gx; p.b_hh = (const __nv_bfloat16*)b_hh;
  p.y = (__nv_bfloat16*)y; p.act = (__nv_bfloat16*)act; p.c_all = c_all; p.counter = counter;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kCols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  int rc = pd_gemm_error_word(&p.err);
  if (rc != PD_OK) return rc;
  CUtensorMap mh, mw;
  rc = pd_make_map_2d(&mh, y, (int64_t)T * Bt, H, H, kBlockK, half ? 64 : 128);
  if (rc != PD_OK) return rc;
  rc = pd_make_map_2d(&mw, w_hh, 4ll * H, H, H, kBlockK, 8);
  if (rc != PD_OK) return rc;
  PD_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned int), s));
  void* args[] = {(void*)&mh, (void*)&mw, (void*)&p};
  PD_CUDA(cudaLaunchCooperativeKernel((const void*)lstm_fwd_persistent_kernel, dim3((unsigned)G), dim3(kThreads), args, smem, s));
  return PD_OK;
}

// Backward recurrence as one cooperative kernel; same return convention as pd_lstm_fwd_persistent.
// dh_ws and dc_ws: fp32 [B, H] scratch each.
int pd_lstm_bwd_persistent(const void* dy, const void* w_hh, const void* act, const float* c_all, int T, int B, int H,
                           void* dgates, float* dh_ws, float* dc_ws, cudaStream_t s) {
  return pd_lstm_bwd_persistent_rows(dy, w_hh, act, c_all, T, B, 0, B, H, dgates, dh_ws, dc_ws, s);
}

// Batch rows b0 .. b0 + B - 1 of tensors with Bt rows per time step (dh_ws, dc_ws: [B, H] of this launch alone).  The
// grid is (H / 128)^2 CTAs - 64 at H = 1024 - so the halves of a batch, launched on two streams, run side by side.
int pd_lstm_bwd_persistent_rows(const void* dy, const void* w_hh, const void* act, const float* c_all, int T, int Bt,
                                int b0, int B, int H, void* dgates, float* dh_ws, float* dc_ws, cudaStream_t s) {
  if (B > 128 || H < kBwdN || H > 1024 || (H & (H - 1)) != 0 || b0 < 0 || b0 + B > Bt) return 1;
  const int NS = H / kBwdN, KS = 4 * H / kBwdK;
  const int G = NS * KS;
  if (H % G != 0 || (H / G) % 8 != 0 || G > pd_num_sms()) return 1;
  const size_t smem = (size_t)kBwdWBytes + (size_t)kBwdStages * kStageBytes + 1024;
  int dev = 0;
  PD_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return 1;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_bwd_state[dev] == 0) {
      int coop = 0, per_sm = 0;
      PD_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
      PD_CUDA(cudaFuncSetAttribute(lstm_bwd_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
      PD_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lstm_bwd_persistent_kernel, kThreads, smem));
      g_bwd_state[dev] = (coop && per_sm >= 1) ? 1 : -1;
    }
    if (g_bwd_state[dev] < 0) return 1;
  }
  unsigned int* counter = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_bwd_counter_base[dev] == nullptr) {
      unsigned int* base = nullptr;
      PD_CUDA(cudaGetSymbolAddress((void**)&base, g_bwd_counters));
      g_bwd_counter_base[dev] = base;
    }
    counter = g_bwd_counter_base[dev] + (g_bwd_next[dev]++ % 64u);
  }
  LstmBwdP p;
  memset(&p, 0, sizeof(p));
  p.T = T; p.B = B; p.H = H; p.G = G; p.U = H / G; p.NS = NS;
  p.Bt = Bt; p.b0 = b0;
  p.dy = (const __nv_bfloat16*)dy; p.act = (const __nv_bfloat16*)act; p.c_all = c_all;
  p.dgates = (__nv_bfloat16*)dgates; p.dh_acc = dh_ws; p.dc = dc_ws; p.counter = counter;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kBwdN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  int rc = pd_gemm_error_word(&p.err);
  if (rc != PD_OK) return rc;
  CUtensorMap mg, mw;
  rc = pd_make_map_2d(&mg, dgates, (int64_t)T * Bt, 4ll * H, 4ll * H, kBlockK, 128);
  if (rc != PD_OK) return rc;
  rc = pd_make_map_2d(&mw, w_hh, 4ll * H, H, H, 64, kBlockK);
  if (rc != PD_OK) return rc;
  PD_CUDA(cudaMemsetAsync(dh_ws, 0, (size_t)B * H * sizeof(float), s));
  PD_CUDA(cudaMemsetAsync(dc_ws, 0, (size_t)B * H * sizeof(float), s));
  PD_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned int), s));
  void* args[] = {(void*)&mg, (void*)&mw, (void*)&p};
  PD_CUDA(cudaLaunchCooperativeKernel((const void*)lstm_bwd_persistent_kernel, dim3((unsigned)G), dim3(kThreads), args, smem, s));
  return PD_OK;
}
