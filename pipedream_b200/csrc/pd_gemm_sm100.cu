// bf16 contraction back end for Blackwell: TMA-fed tcgen05.mma with the fp32
// accumulator in tensor memory.  One CTA computes one 128 x BLOCK_N output tile.
//
//   warp 0   : TMA producer (one elected lane) - fills a ring of shared-memory
//              stages with 128B-swizzled operand boxes
//   warp 1   : allocates tensor memory, issues tcgen05.mma (one elected lane),
//              releases stages through tcgen05.commit
//   warps 2-5: epilogue - tcgen05.ld the accumulator, apply bias / ReLU / border
//              mask, store (or fp32 atomic-add for split-K weight gradients)
//
// Both operands may be K-major (contraction index contiguous in memory) or
// MN-major (output index contiguous); the latter is what lets the data- and
// weight-gradient passes read activations and weights in place, without
// transposed copies.  Convolution taps are extra row offsets of the same 2-D
// tensor maps, so a 3x3 convolution is nine shifted box loads per K-block.
//
// Every mbarrier wait is bounded: when the bound is hit the role records a code
// in an error word, stops, and the CTA still frees its tensor memory.
#include "pd_gemm.cuh"
#include <cuda.h>
#include <mutex>

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;                       // bf16 elements = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kMaxStages = 8;
constexpr uint32_t kABytes = kBlockM * kBlockK * 2;   // 16 KiB
constexpr uint32_t kAtomBytes = 64 * kBlockK * 2;     // one 64-wide MN-major atom: 8 KiB
constexpr long long kWaitCycles = 400000000ll;        // ~0.2 s at 2 GHz

struct KParams {
  int M, N, block_n;
  int num_taps, kb_per_tap, kb_per_split, split_k, num_z;
  int a_major, b_major;
  int a_row0, a_col0, b_row0, b_col0;
  int a_cols, b_cols;
  int a_tap_row[PD_MAX_TAPS], a_tap_col[PD_MAX_TAPS];
  int b_tap_row[PD_MAX_TAPS], b_tap_col[PD_MAX_TAPS];
  int z_b_row[PD_MAX_TAPS];
  long long z_out_col;
  void* out; int out_dtype; long long ldo; int atomic;
  const void* bias; int bias_dtype; int relu;
  int pad_hp, pad_wp;
  const void* relu_aux; long long ld_aux;
  uint32_t idesc;
  int num_stages;
  int* err;
};

__device__ int g_gemm_error = 0;

// ---- PTX wrappers -----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
// Bounded wait: returns false (and records `code`) when the bound runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitCycles) {
      atomicCAS(err, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle.  K-major tiles: rows of 128
// bytes, 8-row groups 1024 bytes apart (SBO).  MN-major tiles: 64-wide atoms of
// kBlockK rows; 8-row K groups 1024 bytes apart (SBO), atoms kAtomBytes apart (LBO).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, int mn_major) {
  const uint32_t lbo = mn_major ? kAtomBytes : 0u;
  const uint32_t sbo = 1024u;
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t tmem_full_bar;
  __shared__ uint32_t tmem_base_holder;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t b_bytes = (uint32_t)p.block_n * kBlockK * 2;
  const uint32_t stage_bytes = kABytes + b_bytes;
  const int S = p.num_stages;

  const int m0 = blockIdx.x * kBlockM;
  const int n0 = blockIdx.y * p.block_n;
  const int z = blockIdx.z / p.split_k;
  const int split = blockIdx.z % p.split_k;
  const int kb_begin = split * p.kb_per_split;
  int kb_end = kb_begin + p.kb_per_split;
  if (kb_end > p.kb_per_tap) kb_end = p.kb_per_tap;
  const int kbn = kb_end - kb_begin;
  const int iters = kbn > 0 ? kbn * p.num_taps : 0;

  // TMEM columns: power of two >= 32 covering block_n
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)p.block_n) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&tmem_full_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_holder)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && iters > 0) {
      const int a_boxes = p.a_major ? 2 : 1;
      const int b_boxes = p.b_major ? p.block_n / 64 : 1;
      for (int it = 0; it < iters; ++it) {
        const int s = it % S;
        const uint32_t ph = (uint32_t)(it / S) & 1u;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, p.err, 1)) break;
        const int t = it / kbn;
        const int kb = kb_begin + it % kbn;
        const uint32_t fb = smem_u32(&full_bar[s]);
        const uint32_t sa = smem0 + (uint32_t)s * stage_bytes;
        const uint32_t sb = sa + kABytes;
        // count the bytes of the boxes that are actually issued
        uint32_t tx = 0;
        int a_issue = 0, b_issue = 0;
        if (p.a_major) {
          for (int j = 0; j < a_boxes; ++j)
            if (p.a_col0 + p.a_tap_col[t] + m0 + j * 64 < p.a_cols) { ++a_issue; tx += kAtomBytes; }
        } else { a_issue = 1; tx += kABytes; }
        if (p.b_major) {
          for (int j = 0; j < b_boxes; ++j)
            if (p.b_col0 + p.b_tap_col[t] + n0 + j * 64 < p.b_cols) { ++b_issue; tx += kAtomBytes; }
        } else { b_issue = 1; tx += b_bytes; }
        mbar_expect_tx(fb, tx);
        if (p.a_major) {
          const int y = p.a_row0 + kb * kBlockK + p.a_tap_row[t];
          for (int j = 0; j < a_issue; ++j)
            tma_load_2d(sa + (uint32_t)j * kAtomBytes, &tma_a, fb, p.a_col0 + p.a_tap_col[t] + m0 + j * 64, y);
        } else {
          tma_load_2d(sa, &tma_a, fb, p.a_col0 + p.a_tap_col[t] + kb * kBlockK, p.a_row0 + m0 + p.a_tap_row[t]);
        }
        if (p.b_major) {
          const int y = p.b_row0 + kb * kBlockK + p.b_tap_row[t] + p.z_b_row[z];
          for (int j = 0; j < b_issue; ++j)
            tma_load_2d(sb + (uint32_t)j * kAtomBytes, &tma_b, fb, p.b_col0 + p.b_tap_col[t] + n0 + j * 64, y);
        } else {
          tma_load_2d(sb, &tma_b, fb, p.b_col0 + p.b_tap_col[t] + kb * kBlockK,
                      p.b_row0 + n0 + p.b_tap_row[t] + p.z_b_row[z]);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && iters > 0) {
      const uint32_t adv_a = p.a_major ? (uint32_t)(kUmmaK * 128) >> 4 : (uint32_t)(kUmmaK * 2) >> 4;
      const uint32_t adv_b = p.b_major ? (uint32_t)(kUmmaK * 128) >> 4 : (uint32_t)(kUmmaK * 2) >> 4;
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % S;
        const uint32_t ph = (uint32_t)(it / S) & 1u;
        ok = mbar_wait(smem_u32(&full_bar[s]), ph, p.err, 2);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t sa = smem0 + (uint32_t)s * stage_bytes;
        const uint64_t da = make_desc(sa, p.a_major);
        const uint64_t db = make_desc(sa + kABytes, p.b_major);
#pragma unroll
        for (int kk = 0; kk < kBlockK / kUmmaK; ++kk)
          umma_bf16(tmem_base, da + (uint64_t)(kk * adv_a), db + (uint64_t)(kk * adv_b), p.idesc,
                    (uint32_t)((it | kk) != 0));
        umma_commit(smem_u32(&empty_bar[s]));
      }
      if (ok) umma_commit(smem_u32(&tmem_full_bar));
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int lg = warp & 3;                 // TMEM lane group this warp may read
    const int m = m0 + lg * 32 + lane;
    bool ready = iters > 0;
    if (ready) ready = mbar_wait(smem_u32(&tmem_full_bar), 0, p.err, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ready) {
      bool border = false;
      if (p.pad_wp > 0) {
        const int wp = m % p.pad_wp;
        const int hp = (m / p.pad_wp) % p.pad_hp;
        border = (wp == 0) | (wp == p.pad_wp - 1) | (hp == 0) | (hp == p.pad_hp - 1);
      }
      const bool row_ok = m < p.M;
      const long long out_col0 = (long long)z * p.z_out_col;
      for (int c0 = 0; c0 < p.block_n; c0 += 32) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld32(tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)c0, r);
        if (!row_ok) continue;
        const int nb = n0 + c0;
        if (nb >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (nb + j < p.N)
              v[j] += p.bias_dtype == PD_BF16 ? __bfloat162float(((const __nv_bfloat16*)p.bias)[nb + j])
                                              : ((const float*)p.bias)[nb + j];
          }
        }
        if (p.relu) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        }
        if (p.relu_aux != nullptr) {
          if (p.out_dtype == PD_BF16) {
            const __nv_bfloat16* ax = (const __nv_bfloat16*)p.relu_aux + (long long)m * p.ld_aux + nb;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nb + j < p.N && !(__bfloat162float(ax[j]) > 0.f)) v[j] = 0.f;
          } else {
            const float* ax = (const float*)p.relu_aux + (long long)m * p.ld_aux + nb;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nb + j < p.N && !(ax[j] > 0.f)) v[j] = 0.f;
          }
        }
        if (border) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        const bool full = nb + 32 <= p.N;
        if (p.atomic) {
          float* o = (float*)p.out + (long long)m * p.ldo + out_col0 + nb;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (full || nb + j < p.N) atomicAdd(o + j, v[j]);
        } else if (p.out_dtype == PD_BF16) {
          __nv_bfloat16* o = (__nv_bfloat16*)p.out + (long long)m * p.ldo + out_col0 + nb;
          if (full && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 pk;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(v[q * 8 + 0], v[q * 8 + 1]);
              __nv_bfloat162 h1 = __floats2bfloat162_rn(v[q * 8 + 2], v[q * 8 + 3]);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(v[q * 8 + 4], v[q * 8 + 5]);
              __nv_bfloat162 h3 = __floats2bfloat162_rn(v[q * 8 + 6], v[q * 8 + 7]);
              pk.x = *reinterpret_cast<uint32_t*>(&h0);
              pk.y = *reinterpret_cast<uint32_t*>(&h1);
              pk.z = *reinterpret_cast<uint32_t*>(&h2);
              pk.w = *reinterpret_cast<uint32_t*>(&h3);
              reinterpret_cast<uint4*>(o)[q] = pk;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nb + j < p.N) o[j] = __float2bfloat16_rn(v[j]);
          }
        } else {
          float* o = (float*)p.out + (long long)m * p.ldo + out_col0 + nb;
          if (full && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              reinterpret_cast<float4*>(o)[q] = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nb + j < p.N) o[j] = v[j];
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---- host side ----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  });
  return fn;
}

int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols,
             int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { pd_set_error("cuTensorMapEncodeTiled is not available from the driver"); return PD_ERR_CUDA; }
  PD_REQUIRE(((uintptr_t)base & 15) == 0, "tcgen05 gemm: operand base must be 16-byte aligned");
  PD_REQUIRE((ld * 2) % 16 == 0, "tcgen05 gemm: leading dimension must be a multiple of 8 elements (got %lld)", (long long)ld);
  PD_REQUIRE(rows > 0 && cols > 0, "tcgen05 gemm: empty operand");
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    pd_set_error("cuTensorMapEncodeTiled failed with code %d (rows=%lld cols=%lld ld=%lld box=%dx%d)", (int)r,
                 (long long)rows, (long long)cols, (long long)ld, box_cols, box_rows);
    return PD_ERR_CUDA;
  }
  return PD_OK;
}

std::mutex g_attr_mu;
bool g_attr_set[64];

}  // namespace

int pd_gemm_pick_block_n(int N, int b_major) {
  int bn;
  if (N > 128) bn = 256;
  else if (N > 64) bn = 128;
  else bn = 64;
  (void)b_major;
  return bn;
}

int pd_gemm_launch_tcgen05(const PdGemm& g, cudaStream_t stream) {
  PD_REQUIRE(g.dtype == PD_BF16, "tcgen05 gemm: operands must be bf16");
  PD_REQUIRE(g.M > 0 && g.N > 0 && g.K > 0, "tcgen05 gemm: empty problem");
  PD_REQUIRE(g.num_taps >= 1 && g.num_taps <= PD_MAX_TAPS, "tcgen05 gemm: bad tap count");
  PD_REQUIRE(g.num_z >= 1 && g.num_z <= PD_MAX_TAPS, "tcgen05 gemm: bad z count");
  PD_REQUIRE(g.split_k >= 1, "tcgen05 gemm: bad split_k");
  PD_REQUIRE(!(g.split_k > 1) || g.atomic, "tcgen05 gemm: split_k needs the atomic epilogue");
  PD_REQUIRE(!g.atomic || g.out_dtype == PD_F32, "tcgen05 gemm: atomic epilogue needs an fp32 output");
  PD_REQUIRE(g.num_taps == 1 || (g.K % kBlockK) == 0, "tcgen05 gemm: multi-tap contraction needs K %% 64 == 0");
  PD_REQUIRE((g.a_col0 % 8) == 0 && (g.b_col0 % 8) == 0, "tcgen05 gemm: column origins must be multiples of 8");
  for (int t = 0; t < g.num_taps; ++t)
    PD_REQUIRE((g.a_tap_col[t] % 8) == 0 && (g.b_tap_col[t] % 8) == 0, "tcgen05 gemm: tap column offsets must be multiples of 8");

  const int block_n = pd_gemm_pick_block_n(g.N, g.b_major);
  KParams p;
  memset(&p, 0, sizeof(p));
  p.M = g.M; p.N = g.N; p.block_n = block_n;
  p.num_taps = g.num_taps;
  p.kb_per_tap = (g.K + kBlockK - 1) / kBlockK;
  p.split_k = g.split_k;
  if (p.split_k > p.kb_per_tap) p.split_k = p.kb_per_tap;
  p.kb_per_split = (p.kb_per_tap + p.split_k - 1) / p.split_k;
  p.split_k = (p.kb_per_tap + p.kb_per_split - 1) / p.kb_per_split;   // no empty splits
  p.num_z = g.num_z;
  p.a_major = g.a_major; p.b_major = g.b_major;
  p.a_row0 = g.a_row0; p.a_col0 = g.a_col0; p.b_row0 = g.b_row0; p.b_col0 = g.b_col0;
  p.a_cols = (int)g.a_cols; p.b_cols = (int)g.b_cols;
  for (int t = 0; t < PD_MAX_TAPS; ++t) {
    p.a_tap_row[t] = g.a_tap_row[t]; p.a_tap_col[t] = g.a_tap_col[t];
    p.b_tap_row[t] = g.b_tap_row[t]; p.b_tap_col[t] = g.b_tap_col[t];
    p.z_b_row[t] = g.z_b_row[t];
  }
  p.z_out_col = g.z_out_col;
  p.out = g.out; p.out_dtype = g.out_dtype; p.ldo = g.ldo; p.atomic = g.atomic;
  p.bias = g.bias; p.bias_dtype = g.bias_dtype; p.relu = g.relu;
  p.pad_hp = g.pad_hp; p.pad_wp = g.pad_wp;
  p.relu_aux = g.relu_aux; p.ld_aux = g.ld_aux;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(g.a_major ? 1 : 0) << 15) |
            ((uint32_t)(g.b_major ? 1 : 0) << 16) | ((uint32_t)(block_n >> 3) << 17) |
            ((uint32_t)(kBlockM >> 4) << 24);
  const uint32_t stage_bytes = kABytes + (uint32_t)block_n * kBlockK * 2;
  int stages = (int)((200u * 1024u) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.num_stages = stages;
  int* err = nullptr;
  PD_CUDA(cudaGetSymbolAddress((void**)&err, g_gemm_error));
  p.err = err;

  CUtensorMap ma, mb;
  int rc = make_map(&ma, g.a, g.a_rows, g.a_cols, g.lda, 64, g.a_major ? kBlockK : kBlockM);
  if (rc != PD_OK) return rc;
  rc = make_map(&mb, g.b, g.b_rows, g.b_cols, g.ldb, 64, g.b_major ? kBlockK : block_n);
  if (rc != PD_OK) return rc;

  const size_t smem = (size_t)stages * stage_bytes + 1024;
  {
    int dev = 0;
    PD_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_attr_mu);
    if (dev >= 0 && dev < 64 && !g_attr_set[dev]) {
      PD_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
      g_attr_set[dev] = true;
    }
  }
  dim3 grid((g.M + kBlockM - 1) / kBlockM, (g.N + block_n - 1) / block_n, g.num_z * p.split_k);
  gemm_tcgen05_kernel<<<grid, kThreads, smem, stream>>>(ma, mb, p);
  PD_LAUNCH_CHECK("gemm_tcgen05_kernel");
  return PD_OK;
}

// Reads and clears the device-side error word of the tcgen05 kernels
// (0 = none, 1/2/3 = producer / MMA / epilogue wait ran out).  Synchronises.
PD_EXPORT int pd_gemm_poll_error(int* code) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(code, "pd_gemm_poll_error: null output");
  int v = 0;
  PD_CUDA(cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    PD_CUDA(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
  }
  *code = v;
  return PD_OK;
}
