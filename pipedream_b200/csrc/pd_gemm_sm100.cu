// bf16 contraction back end for Blackwell: TMA-fed tcgen05.mma with the fp32
// accumulator in tensor memory.  One CTA computes one 128 x BLOCK_N output tile.
//
//   warp 0    : TMA producer (one elected lane) - fills a ring of shared-memory
//               stages with 128B-swizzled operand boxes
//   warp 1    : allocates tensor memory, issues tcgen05.mma (one elected lane),
//               releases stages through tcgen05.commit
//   warp 2    : second MMA issuer, used by narrow tiles (two 128-row groups per tile)
//   warps 3-10: epilogue, two sets of four warps - tcgen05.ld the accumulator, apply
//               bias / ReLU / border mask, store (or fp32 atomic-add for split-K weight
//               gradients); the sets take alternate tiles, or one group each
//
// Both operands may be K-major (contraction index contiguous in memory) or
// MN-major (output index contiguous); the latter is what lets the data- and
// weight-gradient passes read activations and weights in place, without
// transposed copies.  Convolution taps are extra row offsets of the same 2-D
// tensor maps, so a 3x3 convolution is nine shifted box loads per K-block - or, for narrow layers that are
// bound by shared-memory fill bandwidth rather than by the tensor pipe, three boxes of 136 rows, each read by
// the three taps of one filter row through descriptors that start 0, 1 or 2 rows into the box.
//
// Wide problems (output tile 256 x 256) run the same roles on a pair of CTAs (cluster of two, cta_group::2): a
// tcgen05.mma costs about 150 cycles to issue whatever its shape, so only N = 256 instructions can keep the
// tensor pipe busy, and the pair halves the operand bytes each SM has to pull in per FLOP (each CTA loads its
// own 128 rows of A and its half of B; the even CTA issues the MMAs for both and signals the barriers of both).
//
// Every mbarrier wait is bounded: when the bound is hit the role records a code
// in an error word, stops, and the CTA still frees its tensor memory.
#include "pd_gemm.cuh"
#include "pd_sm100_ptx.cuh"
#include <cuda.h>
#include <mutex>
#include <cstdlib>

namespace {

using namespace pd_sm100;

constexpr int kBlockM = 128;
constexpr int kUmmaK = 16;
constexpr int kThreads = 352;                     // producer, 2 MMA issuers, 2 x 4 epilogue warps
constexpr int kEpiWarp0 = 3;                      // first epilogue warp
constexpr int kMaxAccBufs = 4;
constexpr int kMaxStages = 8;
constexpr uint32_t kABytes = kBlockM * kBlockK * 2;   // 16 KiB
constexpr int kBox3Rows = kBlockM + 8;                 // A box shared by the three taps of one filter row
constexpr uint32_t kA3Bytes = kBox3Rows * kBlockK * 2; // 17 KiB (a multiple of 1024)

struct KParams {
  int M, N, block_n, m_tiles, n_tiles;
  int groups;                 // 128-row sub-tiles of a tile, each with its own MMA issuer warp, accumulators and epilogue set
  int cta_n;                  // B rows (columns of the output tile) one CTA loads: block_n, or half of it for a CTA pair
  int num_taps, kb_per_tap, kb_per_split, split_k, num_z;   // num_z = number of z groups
  int acc_count, num_z_total;                                // accumulators per tile, outputs in all
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
  int acc_bufs;               // accumulator buffers in tensor memory (2..4): tiles in flight between MMA and epilogue
  // tap3: the taps come in triples whose A rows differ by 0/1/2 (the three taps of one filter row of a 3x3
  // convolution): one A box of kBox3Rows rows serves all three, num_taps counts triples
  int tap3;
  int t3_base[3], t3_off[PD_MAX_TAPS];
  // divisions of the per-tile bookkeeping as multiply-high + shift (see fast_div): a 32-bit division is a chain of
  // some twenty dependent instructions, and the single MMA-issuing thread runs every one of them between two tiles
  uint32_t fd_tiles_mn[2], fd_n_tiles[2], fd_num_z[2], fd_pad_wp[2], fd_pad_hp[2];
  int* err;
  long long* stall;           // diagnostic (may be null): per CTA {cycles waiting for operands, for a free accumulator, total, tiles}
};

__device__ int g_gemm_error = 0;

// n / d for 0 <= n < 2^31 with d's pair {multiplier, shift} from make_fast_div (multiplier 0 stands for d == 1).
__device__ __forceinline__ int fast_div(int n, const uint32_t* fd) {
  return fd[0] ? (int)(__umulhi((uint32_t)n, fd[0]) >> fd[1]) : n;
}

// Epilogue of one 32-column chunk of one accumulator row: bias, ReLU, masks, store / atomic add.
__device__ __forceinline__ void epilogue_chunk(const KParams& p, const uint32_t* r, int m, int nb, long long out_col0,
                                               bool border) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (p.bias != nullptr) {
    const __nv_bfloat16* bb = (const __nv_bfloat16*)p.bias + nb;
    if (p.bias_dtype == PD_BF16 && nb + 32 <= p.N && (((uintptr_t)bb) & 15) == 0) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 pk = __ldg(reinterpret_cast<const uint4*>(bb) + q);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          v[q * 8 + 2 * e] += f.x;
          v[q * 8 + 2 * e + 1] += f.y;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (nb + j < p.N)
          v[j] += p.bias_dtype == PD_BF16 ? __bfloat162float(((const __nv_bfloat16*)p.bias)[nb + j])
                                          : ((const float*)p.bias)[nb + j];
      }
    }
  }
  if (p.relu) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
  }
  if (p.relu_aux != nullptr) {
    if (p.out_dtype == PD_BF16) {
      const __nv_bfloat16* ax = (const __nv_bfloat16*)p.relu_aux + (long long)m * p.ld_aux + nb;
      if (nb + 32 <= p.N && (((uintptr_t)ax) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 pk = reinterpret_cast<const uint4*>(ax)[q];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            if (!(f.x > 0.f)) v[q * 8 + 2 * e] = 0.f;
            if (!(f.y > 0.f)) v[q * 8 + 2 * e + 1] = 0.f;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (nb + j < p.N && !(__bfloat162float(ax[j]) > 0.f)) v[j] = 0.f;
      }
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
    if (full && (((uintptr_t)o) & 15) == 0) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                     ::"l"(o + q * 4), "f"(v[q * 4]), "f"(v[q * 4 + 1]), "f"(v[q * 4 + 2]), "f"(v[q * 4 + 3])
                     : "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (full || nb + j < p.N) atomicAdd(o + j, v[j]);
    }
  } else if (p.out_dtype == PD_BF16) {
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (long long)m * p.ldo + out_col0 + nb;
    if (full && (((uintptr_t)o) & 31) == 0) {
      // 32-byte stores: a lane writes whole sectors, so the two halves of a sector do not travel separately
      uint32_t w[16];
#pragma unroll
      for (int q = 0; q < 16; ++q) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
        w[q] = *reinterpret_cast<uint32_t*>(&h);
      }
#pragma unroll
      for (int q = 0; q < 2; ++q)
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"l"(o + q * 16), "r"(w[q * 8]), "r"(w[q * 8 + 1]), "r"(w[q * 8 + 2]), "r"(w[q * 8 + 3]),
                       "r"(w[q * 8 + 4]), "r"(w[q * 8 + 5]), "r"(w[q * 8 + 6]), "r"(w[q * 8 + 7])
                     : "memory");
    } else if (full && (((uintptr_t)o) & 15) == 0) {
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
    if (full && (((uintptr_t)o) & 31) == 0) {
      // 32-byte stores, as for bf16 above (a weight gradient with a short contraction - a Linear layer at batch 64 -
      // is all epilogue: 128 KiB of fp32 per tile for four MMAs)
#pragma unroll
      for (int q = 0; q < 4; ++q)
        asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"l"(o + q * 8), "r"(__float_as_uint(v[q * 8])), "r"(__float_as_uint(v[q * 8 + 1])),
                       "r"(__float_as_uint(v[q * 8 + 2])), "r"(__float_as_uint(v[q * 8 + 3])),
                       "r"(__float_as_uint(v[q * 8 + 4])), "r"(__float_as_uint(v[q * 8 + 5])),
                       "r"(__float_as_uint(v[q * 8 + 6])), "r"(__float_as_uint(v[q * 8 + 7]))
                     : "memory");
    } else if (full && (((uintptr_t)o) & 15) == 0) {
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

template <int CG>
__device__ __forceinline__ void umma_cg(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  if constexpr (CG == 1) umma_bf16(tmem_d, da, db, idesc, acc);
  else umma_bf16_pair(tmem_d, da, db, idesc, acc);
}
template <int CG>
__device__ __forceinline__ void commit_cg(uint32_t bar) {
  if constexpr (CG == 1) umma_commit(bar);
  else umma_commit_pair(bar);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Persistent: each CTA walks the tile list with stride gridDim.x.  Tensor memory holds 2..4 accumulator
// buffers, so the epilogues of earlier tiles (two warp sets, alternate tiles) run under the MMAs of the
// next ones - short-K tiles are bound by the epilogue's latency chain otherwise; the shared-memory stage
// ring runs on across tile boundaries.
//
// CG = 2: the CTAs of a cluster of two share one 256-row tile.  Rank 0 ("leader") owns the barriers the MMA
// issuer waits on: both producers' TMA loads complete on the leader's full barrier, both CTAs' epilogue warps
// arrive on the leader's tmem_empty barrier; the leader's commits arrive on the empty / tmem_full barriers of
// both CTAs.
template <int CG>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages];
  __shared__ __align__(8) uint64_t empty_bar[kMaxStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[2 * kMaxAccBufs];     // [group][buffer]
  __shared__ __align__(8) uint64_t tmem_empty_bar[2 * kMaxAccBufs];
  __shared__ uint32_t tmem_base_holder;

  // broadcast from lane 0 so that the compiler knows the warp index is the same in every lane of a warp: the role
  // branches below are then warp-uniform and the code inside them can use the uniform datapath
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t rank = CG == 2 ? cluster_ctarank() : 0u;   // position in the CTA pair
  const bool leader = rank == 0u;
  // Each CTA (CG = 1) or pair (CG = 2) walks the tile list with a stride of the number of CTAs / pairs.  The loop is
  // written on blockIdx / gridDim directly: routed through local copies the same loop compiled into a kernel whose
  // MMA issue interval was a fifth longer (measured on every layer shape).
#define PD_FIRST_TILE (CG == 1 ? blockIdx.x : (blockIdx.x >> 1))
#define PD_TILE_STEP (CG == 1 ? gridDim.x : (gridDim.x >> 1))
  const uint32_t b_bytes = (uint32_t)p.cta_n * kBlockK * 2;
  const int G = p.groups;
  const uint32_t a_bytes = p.tap3 ? kA3Bytes : kABytes;      // one group's A box
  const uint32_t a_total = (uint32_t)G * a_bytes;            // B tiles follow the groups' A boxes in a stage
  const uint32_t stage_bytes = a_total + (p.tap3 ? 3u : (uint32_t)p.acc_count) * b_bytes;
  const int group_rows = kBlockM * CG;                       // rows between the groups of a tile
  const int S = p.num_stages;
  const uint32_t acc_cols = (uint32_t)(p.acc_count * p.block_n);   // TMEM columns of one buffer
  const int tiles_mn = p.m_tiles * p.n_tiles;
  const int total_tiles = tiles_mn * p.num_z * p.split_k;

  // TMEM columns: power of two >= 32 covering all accumulator buffers
  const uint32_t nbuf = (uint32_t)p.acc_bufs;
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)G * nbuf * acc_cols) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), (uint32_t)G);    // one commit per issuer
    }
    for (int b = 0; b < 2 * kMaxAccBufs; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 4 * CG);     // one arrival per epilogue warp (of both CTAs of a pair)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (CG == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(&tmem_base_holder)), "r"(tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(&tmem_base_holder)), "r"(tmem_cols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();     // the peer's barriers exist before anything is signalled on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_holder;

  // tile -> (m0, n0, z, kb_begin, kbn); n varies fastest so that CTAs running together share A rows
#define PD_DECODE_TILE(tile)                                                   \
  const int zs_ = fast_div((tile), p.fd_tiles_mn);                             \
  const int rem_ = (tile) - zs_ * tiles_mn;                                    \
  const int mt_ = fast_div(rem_, p.fd_n_tiles);                                \
  const int m0 = mt_ * (kBlockM * CG * G) + (int)rank * kBlockM;               \
  const int n0 = (rem_ - mt_ * p.n_tiles) * p.block_n;                         \
  const int n0l = n0 + (int)rank * p.cta_n;  /* first B row this CTA loads */  \
  /* z varies faster than the K slice: the z outputs of a weight gradient (filter taps) read the same      \
     activation rows shifted by a pixel or a row, so running them side by side fetches those rows from   \
     HBM once and serves the other taps from L2 */                                                         \
  const int ks_ = fast_div(zs_, p.fd_num_z);                                   \
  const int z = zs_ - ks_ * p.num_z;                                           \
  const int kb_begin = ks_ * p.kb_per_split;                                   \
  const int kb_end_ = min(kb_begin + p.kb_per_split, p.kb_per_tap);            \
  const int kbn = kb_end_ - kb_begin;                                          \
  const int iters = kbn > 0 ? kbn * p.num_taps : 0;                             \
  const int acc0 = z * p.acc_count;                                             \
  const int accn = min(p.acc_count, p.num_z_total - acc0);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The whole warp walks the loop; lane 0 arms the barrier, lanes 0..boxes-1 each issue one box,
    // so the (up to six) box loads of a stage go out in one instruction slot.
    // Two boxes per stage (both operands K-major): one lane issues both, nothing to coordinate.
    if (p.tap3) {
      // lanes 0..G-1: the shared A box of each group; the lanes after them: the B boxes of the triple's three taps
      const int b_boxes = p.b_major ? p.cta_n / 64 : 1;
      const bool is_a = lane < G;
      const int bl = lane - G;
      const int s3 = is_a ? 0 : min(bl / b_boxes, 2);
      const int j = is_a ? 0 : bl % b_boxes;
      const bool has_box = is_a || bl < 3 * b_boxes;
      uint32_t g = 0;
      bool ok = true;
      for (int tile = PD_FIRST_TILE; tile < total_tiles && ok; tile += PD_TILE_STEP) {
        PD_DECODE_TILE(tile)
        (void)iters; (void)accn; (void)acc0; (void)z; (void)n0;
        for (int r = 0; r < 3 && ok; ++r) {
          int x0, y0, xk, yk;
          uint32_t dst_off, bytes;
          bool issue = has_box;
          if (is_a) {
            x0 = p.a_col0; y0 = p.a_row0 + m0 + lane * group_rows + p.t3_base[r]; xk = kBlockK; yk = 0;
            dst_off = (uint32_t)lane * kA3Bytes; bytes = kA3Bytes;
          } else {
            const int t = 3 * r + s3;
            if (p.b_major) {
              x0 = p.b_col0 + p.b_tap_col[t] + n0l + j * 64; y0 = p.b_row0 + p.b_tap_row[t]; xk = 0; yk = kBlockK;
              dst_off = a_total + (uint32_t)s3 * b_bytes + (uint32_t)j * kAtomBytes; bytes = kAtomBytes;
              if (CG == 1) issue = issue && x0 < p.b_cols;
            } else {
              x0 = p.b_col0 + p.b_tap_col[t]; y0 = p.b_row0 + n0l + p.b_tap_row[t]; xk = kBlockK; yk = 0;
              dst_off = a_total + (uint32_t)s3 * b_bytes; bytes = b_bytes;
            }
          }
          uint32_t tx = issue ? bytes : 0u;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
          const CUtensorMap* map = is_a ? &tma_a : &tma_b;
          for (int kb = kb_begin; kb < kb_begin + kbn; ++kb, ++g) {
            const int s = (int)(g % (uint32_t)S);
            const uint32_t ph = (g / (uint32_t)S) & 1u;
            if (lane == 0) ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, p.err, 1);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) break;
            const uint32_t fb = smem_u32(&full_bar[s]);
            if (lane == 0 && leader) mbar_expect_tx(fb, tx * CG);    // the peer's boxes land on the same barrier
            __syncwarp();
            if (issue) {
              if constexpr (CG == 1)
                tma_load_2d(smem0 + (uint32_t)s * stage_bytes + dst_off, map, fb, x0 + kb * xk, y0 + kb * yk);
              else
                tma_load_2d_pair(smem0 + (uint32_t)s * stage_bytes + dst_off, map, mapa_shared(fb, 0), x0 + kb * xk,
                                 y0 + kb * yk);
            }
          }
        }
      }
    } else if (!p.a_major && !p.b_major && p.acc_count == 1) {
      if (lane == 0) {
        uint32_t g = 0;
        bool ok = true;
        for (int tile = PD_FIRST_TILE; tile < total_tiles && ok; tile += PD_TILE_STEP) {
          PD_DECODE_TILE(tile)
          (void)iters; (void)accn; (void)n0;
          const int zrow = p.z_b_row[min(acc0, PD_MAX_TAPS - 1)];
          for (int t = 0; t < p.num_taps && ok; ++t) {
            const int ax = p.a_col0 + p.a_tap_col[t], ay = p.a_row0 + m0 + p.a_tap_row[t];
            const int bx = p.b_col0 + p.b_tap_col[t], by = p.b_row0 + n0l + p.b_tap_row[t] + zrow;
            for (int kb = kb_begin; kb < kb_begin + kbn; ++kb, ++g) {
              const int s = (int)(g % (uint32_t)S);
              const uint32_t ph = (g / (uint32_t)S) & 1u;
              if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, p.err, 1)) { ok = false; break; }
              const uint32_t fb = smem_u32(&full_bar[s]);
              const uint32_t sa = smem0 + (uint32_t)s * stage_bytes;
              if (leader) mbar_expect_tx(fb, (a_total + b_bytes) * CG);
              if constexpr (CG == 1) {
                for (int g = 0; g < G; ++g)
                  tma_load_2d(sa + (uint32_t)g * kABytes, &tma_a, fb, ax + kb * kBlockK, ay + g * group_rows);
                tma_load_2d(sa + a_total, &tma_b, fb, bx + kb * kBlockK, by);
              } else {
                const uint32_t fbc = mapa_shared(fb, 0);
                for (int g = 0; g < G; ++g)
                  tma_load_2d_pair(sa + (uint32_t)g * kABytes, &tma_a, fbc, ax + kb * kBlockK, ay + g * group_rows);
                tma_load_2d_pair(sa + a_total, &tma_b, fbc, bx + kb * kBlockK, by);
              }
            }
          }
        }
      }
    } else
    {
      const int a_boxes = p.a_major ? 2 : 1;                 // per group
      const int b_boxes = p.b_major ? p.cta_n / 64 : 1;
      const bool is_a = lane < a_boxes * G;
      const int ag = is_a ? lane / a_boxes : 0;              // A lanes: which group's tile
      const int bl = lane - a_boxes * G;                     // B lanes: accumulator-major
      const int acc = is_a ? 0 : bl / b_boxes;               // which accumulator's B tile
      const int j = is_a ? lane % a_boxes : bl % b_boxes;    // box index within its operand tile
      uint32_t g = 0;                       // stage uses so far (ring position across tiles)
      bool ok = true;
      for (int tile = PD_FIRST_TILE; tile < total_tiles && ok; tile += PD_TILE_STEP) {
        PD_DECODE_TILE(tile)
        (void)iters; (void)n0;
        const bool has_box = is_a || acc < accn;
        const int zrow = p.z_b_row[min(acc0 + acc, PD_MAX_TAPS - 1)];
        for (int t = 0; t < p.num_taps && ok; ++t) {
          // per-tap constants of this lane's box
          int x0, y0, xk, yk;              // coordinate = (x0 + kb * xk, y0 + kb * yk)
          uint32_t dst_off, bytes;
          bool issue = has_box;
          if (is_a) {
            if (p.a_major) {
              x0 = p.a_col0 + p.a_tap_col[t] + m0 + ag * group_rows + j * 64; y0 = p.a_row0 + p.a_tap_row[t]; xk = 0; yk = kBlockK;
              dst_off = (uint32_t)ag * kABytes + (uint32_t)j * kAtomBytes; bytes = kAtomBytes;
              if (CG == 1) issue = issue && x0 < p.a_cols;
            } else {
              x0 = p.a_col0 + p.a_tap_col[t]; y0 = p.a_row0 + m0 + ag * group_rows + p.a_tap_row[t]; xk = kBlockK; yk = 0;
              dst_off = (uint32_t)ag * kABytes; bytes = kABytes;
            }
          } else {
            if (p.b_major) {
              x0 = p.b_col0 + p.b_tap_col[t] + n0l + j * 64; y0 = p.b_row0 + p.b_tap_row[t] + zrow; xk = 0; yk = kBlockK;
              dst_off = a_total + (uint32_t)acc * b_bytes + (uint32_t)j * kAtomBytes; bytes = kAtomBytes;
              if (CG == 1) issue = issue && x0 < p.b_cols;
            } else {
              x0 = p.b_col0 + p.b_tap_col[t]; y0 = p.b_row0 + n0l + p.b_tap_row[t] + zrow; xk = kBlockK; yk = 0;
              dst_off = a_total + (uint32_t)acc * b_bytes; bytes = b_bytes;
            }
          }
          // bytes that will land in a stage = sum over the issuing lanes
          uint32_t tx = issue ? bytes : 0u;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) tx += __shfl_xor_sync(0xffffffffu, tx, o);
          const CUtensorMap* map = is_a ? &tma_a : &tma_b;
          for (int kb = kb_begin; kb < kb_begin + kbn; ++kb, ++g) {
            const int s = (int)(g % (uint32_t)S);
            const uint32_t ph = (g / (uint32_t)S) & 1u;
            if (lane == 0) ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1u, p.err, 1);
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) break;
            const uint32_t fb = smem_u32(&full_bar[s]);
            if (lane == 0 && leader) mbar_expect_tx(fb, tx * CG);    // the peer's boxes land on the same barrier
            __syncwarp();
            if (issue) {
              if constexpr (CG == 1)
                tma_load_2d(smem0 + (uint32_t)s * stage_bytes + dst_off, map, fb, x0 + kb * xk, y0 + kb * yk);
              else
                tma_load_2d_pair(smem0 + (uint32_t)s * stage_bytes + dst_off, map, mapa_shared(fb, 0), x0 + kb * xk,
                                 y0 + kb * yk);
            }
          }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ------------------------------- MMA issuers ------------------------------
    // One warp per group; one lane issues.  The issuing thread runs every instruction between two MMAs itself, and a
    // tcgen05.mma is only 32 (N = 64) to 128 (N = 256) cycles of tensor-pipe work, so the loops below are kept to a
    // handful of instructions per MMA: descriptors are advanced by 32-bit adds on their low words, the ring position
    // and its barrier addresses are carried along instead of being derived by division, and nothing is decided per
    // MMA that can be decided per tile.  Narrow tiles (N <= 128) still need two issuers to fill the pipe - each
    // with its own accumulators and A rows, sharing the stage's B tiles.
    const int grp = warp - 1;
    if (lane == 0 && leader && grp < G) {
      const uint32_t bar0 = (uint32_t)grp * kMaxAccBufs;           // this group's tmem barriers
      const uint32_t tmem_g = tmem_base + (uint32_t)grp * nbuf * acc_cols;
      const uint32_t adv_a = p.a_major ? (uint32_t)(kUmmaK * 128) >> 4 : (uint32_t)(kUmmaK * 2) >> 4;
      const uint32_t adv_b = p.b_major ? (uint32_t)(kUmmaK * 128) >> 4 : (uint32_t)(kUmmaK * 2) >> 4;
      constexpr int kSteps = kBlockK / kUmmaK;
      // descriptor words of stage 0; a stage further on adds stage_lo to the low words
      const uint64_t da0 = make_desc(smem0 + (uint32_t)grp * a_bytes, p.a_major);
      const uint64_t db0 = make_desc(smem0 + a_total, p.b_major);
      const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
      const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
      const uint32_t stage_lo = stage_bytes >> 4;
      const uint32_t b_tile_lo = b_bytes >> 4;
      const uint32_t full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
      const uint32_t idesc = p.idesc;
      // ring position, carried across tiles
      int s = 0;
      uint32_t ph = 0, a_lo = a_lo0, b_lo = b_lo0, fb = full0, eb = empty0;
#define PD_NEXT_STAGE                                                         \
      ++s; a_lo += stage_lo; b_lo += stage_lo; fb += 8; eb += 8;                \
      if (s == S) { s = 0; ph ^= 1u; a_lo = a_lo0; b_lo = b_lo0; fb = full0; eb = empty0; }
      uint32_t local = 0;                   // tiles done by this CTA
      uint32_t buf = 0, use = 0;            // local % nbuf and the parity of local / nbuf, carried along
      bool ok = true;
      const bool timing = p.stall != nullptr;
      long long t_ops = 0, t_acc = 0;
      const long long t_begin = timing ? clock64() : 0;
      for (int tile = PD_FIRST_TILE; tile < total_tiles && ok; tile += PD_TILE_STEP) {
        PD_DECODE_TILE(tile)
        (void)m0; (void)n0; (void)n0l; (void)kb_begin; (void)acc0;
        if (iters == 0) continue;             // (cannot happen: the host never creates empty splits)
        // the epilogue must have drained this accumulator (passes at once on its first use)
        const long long ta = timing ? clock64() : 0;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[bar0 + buf]), (use & 1u) ^ 1u, p.err, 4);
        if (timing) t_acc += clock64() - ta;
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_g + buf * acc_cols;
        uint32_t acc = 0;                     // the tile's first MMA overwrites the accumulator
        if (p.tap3) {
          for (int r = 0; r < 3 && ok; ++r) {
            // the taps' rows start t3_off (0..2) rows into the shared box; the swizzle is a function of the
            // shared-memory address, so a descriptor may start on any 128-byte row of the box
            const uint32_t o0 = (uint32_t)p.t3_off[3 * r] * 8u, o1 = (uint32_t)p.t3_off[3 * r + 1] * 8u,
                           o2 = (uint32_t)p.t3_off[3 * r + 2] * 8u;
            for (int kb = 0; kb < kbn; ++kb) {
              const long long tw = timing ? clock64() : 0;
              ok = mbar_wait(fb, ph, p.err, 2);
              if (timing) t_ops += clock64() - tw;
              if (!ok) break;
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              umma_lo<CG, 2>(tmem_d, a_lo + o0, a_hi, b_lo, b_hi, idesc, acc);
#pragma unroll
              for (int kk = 1; kk < kSteps; ++kk)
                umma_lo<CG, 1>(tmem_d, a_lo + o0 + kk * adv_a, a_hi, b_lo + kk * adv_b, b_hi, idesc, 1u);
#pragma unroll
              for (int kk = 0; kk < kSteps; ++kk)
                umma_lo<CG, 1>(tmem_d, a_lo + o1 + kk * adv_a, a_hi, b_lo + b_tile_lo + kk * adv_b, b_hi, idesc, 1u);
#pragma unroll
              for (int kk = 0; kk < kSteps; ++kk)
                umma_lo<CG, 1>(tmem_d, a_lo + o2 + kk * adv_a, a_hi, b_lo + 2u * b_tile_lo + kk * adv_b, b_hi, idesc, 1u);
              commit_cg<CG>(eb);
              acc = 1u;
              PD_NEXT_STAGE
            }
          }
        } else if (p.b_major && accn > 1 && accn * p.block_n <= 256) {
          // MN-major B tiles of the accumulators of a z group lie back to back, 64-column atom after atom,
          // and so do their accumulators in tensor memory: one MMA of N = accn * block_n does the work of
          // accn narrow ones
          const uint32_t idesc_n = (idesc & ~(0x3Fu << 17)) | ((uint32_t)((accn * p.block_n) >> 3) << 17);
          for (int it = 0; it < iters; ++it) {
            const long long tw = timing ? clock64() : 0;
            ok = mbar_wait(fb, ph, p.err, 2);
            if (timing) t_ops += clock64() - tw;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            umma_lo<CG, 2>(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc_n, acc);
#pragma unroll
            for (int kk = 1; kk < kSteps; ++kk)
              umma_lo<CG, 1>(tmem_d, a_lo + kk * adv_a, a_hi, b_lo + kk * adv_b, b_hi, idesc_n, 1u);
            commit_cg<CG>(eb);
            acc = 1u;
            PD_NEXT_STAGE
          }
        } else {
          for (int it = 0; it < iters; ++it) {
            const long long tw = timing ? clock64() : 0;
            ok = mbar_wait(fb, ph, p.err, 2);
            if (timing) t_ops += clock64() - tw;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int a = 0; a < accn; ++a) {
              const uint32_t tmem_a = tmem_d + (uint32_t)(a * p.block_n);
              const uint32_t b_lo_a = b_lo + (uint32_t)a * b_tile_lo;
              umma_lo<CG, 2>(tmem_a, a_lo, a_hi, b_lo_a, b_hi, idesc, acc);
#pragma unroll
              for (int kk = 1; kk < kSteps; ++kk)
                umma_lo<CG, 1>(tmem_a, a_lo + kk * adv_a, a_hi, b_lo_a + kk * adv_b, b_hi, idesc, 1u);
            }
            commit_cg<CG>(eb);
            acc = 1u;
            PD_NEXT_STAGE
          }
        }
        if (ok) commit_cg<CG>(smem_u32(&tmem_full_bar[bar0 + buf]));
        ++local;
        if (++buf == nbuf) { buf = 0; use ^= 1u; }
      }
#undef PD_NEXT_STAGE
      if (timing && grp == 0) {
        long long* o = p.stall + 4ll * blockIdx.x;
        o[0] += t_ops; o[1] += t_acc; o[2] += clock64() - t_begin; o[3] += local;
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int lg = warp & 3;                 // TMEM lane group this warp may read
    const uint32_t set = (uint32_t)(warp - kEpiWarp0) >> 2;   // which of the two epilogue sets
    // one group: the sets take alternate tiles; two groups: each set drains its own group's accumulators
    const uint32_t grp = G == 2 ? set : 0u;
    const uint32_t bar0 = grp * kMaxAccBufs;
    uint32_t local = 0;
    uint32_t buf = 0, use = 0;              // local % nbuf and the parity of local / nbuf
    bool ok = true;
#define PD_NEXT_LOCAL ++local; if (++buf == nbuf) { buf = 0; use ^= 1u; }
    for (int tile = PD_FIRST_TILE; tile < total_tiles && ok; tile += PD_TILE_STEP) {
      PD_DECODE_TILE(tile)
      (void)kb_begin; (void)n0l;
      if (iters == 0) continue;
      if (G == 1 && (local & 1u) != set) { PD_NEXT_LOCAL continue; }
      ok = mbar_wait(smem_u32(&tmem_full_bar[bar0 + buf]), use & 1u, p.err, 3);
      // the wait result can differ between lanes only when the bound ran out; make it uniform
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = m0 + (int)grp * group_rows + lg * 32 + lane;
      bool border = false;
      if (p.pad_wp > 0) {
        const int row_ = fast_div(m, p.fd_pad_wp);
        const int wp = m - row_ * p.pad_wp;
        const int hp = row_ - fast_div(row_, p.fd_pad_hp) * p.pad_hp;
        border = (wp == 0) | (wp == p.pad_wp - 1) | (hp == 0) | (hp == p.pad_hp - 1);
      }
      const bool row_ok = m < p.M;
      const uint32_t tmem_acc = tmem_base + (grp * nbuf + buf) * acc_cols + ((uint32_t)(lg * 32) << 16);
      const int total_cols = accn * p.block_n;
      for (int cc = 0; cc < total_cols; cc += 64) {
        // two chunks in flight per wait
        const bool two = cc + 32 < total_cols;
        uint32_t r0[32], r1[32];
        __syncwarp();
        tmem_ld32(tmem_acc + (uint32_t)cc, r0);
        if (two) tmem_ld32(tmem_acc + (uint32_t)(cc + 32), r1);
        tmem_ld_wait();
        if (cc + 64 >= total_cols) {
          // the accumulator is in registers now: hand it back to the MMA warp before the arithmetic and the stores
          // of this last pair of chunks (an arrive after them would also wait for the stores to be performed)
          __syncwarp();
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          if (lane == 0) {
            if (leader) mbar_arrive(smem_u32(&tmem_empty_bar[bar0 + buf]));
            else mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty_bar[bar0 + buf]), 0));
          }
        }
        if (row_ok) {
          {
            const int a = accn == 1 ? 0 : cc / p.block_n, c0 = cc - a * p.block_n;
            if (n0 + c0 < p.N) epilogue_chunk(p, r0, m, n0 + c0, (long long)(acc0 + a) * p.z_out_col, border);
          }
          if (two) {
            const int a = accn == 1 ? 0 : (cc + 32) / p.block_n, c0 = cc + 32 - a * p.block_n;
            if (n0 + c0 < p.N) epilogue_chunk(p, r1, m, n0 + c0, (long long)(acc0 + a) * p.z_out_col, border);
          }
        }
      }
      PD_NEXT_LOCAL
    }
#undef PD_NEXT_LOCAL
  }
#undef PD_DECODE_TILE
#undef PD_FIRST_TILE
#undef PD_TILE_STEP

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  // a pair stays together until both are done: the leader's MMAs read the peer's shared memory and write its
  // tensor memory, and the peer's last arrivals land on the leader's barriers
  if constexpr (CG == 2) cluster_sync_all();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (CG == 1)
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---- host side ----------------------------------------------------------------
// {multiplier, shift} with n / d == umulhi(n, multiplier) >> shift for every 0 <= n < 2^31 (d >= 1; d == 1 is coded as
// multiplier 0): multiplier = ceil(2^(31 + ceil(log2 d)) / d), which fits 32 bits, shift = ceil(log2 d) - 1.
void make_fast_div(uint32_t d, uint32_t* fd) {
  if (d <= 1) { fd[0] = 0; fd[1] = 0; return; }
  uint32_t lg = 0;
  while ((1ull << lg) < d) ++lg;
  const uint64_t pw = 1ull << (31 + lg);
  fd[0] = (uint32_t)((pw + d - 1) / d);
  fd[1] = lg - 1;
}

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

// Encoded tensor maps are cached per host thread: the time loop of an LSTM layer launches the same
// two maps once per step (only the row coordinate moves), and encoding costs more than the launch.
struct MapKey {
  const void* base; int64_t rows, cols, ld; int box_cols, box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_cols == o.box_cols && box_rows == o.box_rows;
  }
};
struct MapCache {
  static constexpr int kEntries = 16;
  MapKey key[kEntries];
  CUtensorMap map[kEntries];
  bool valid[kEntries] = {};
  int next = 0;
};
thread_local MapCache g_map_cache;

}  // namespace

int pd_make_map_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_cols,
                   int box_rows) {
  const MapKey k{base, rows, cols, ld, box_cols, box_rows};
  MapCache& c = g_map_cache;
  for (int i = 0; i < MapCache::kEntries; ++i)
    if (c.valid[i] && c.key[i] == k) { *map = c.map[i]; return PD_OK; }
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
  c.key[c.next] = k; c.map[c.next] = *map; c.valid[c.next] = true;
  c.next = (c.next + 1) % MapCache::kEntries;
  return PD_OK;
}

namespace {

std::mutex g_attr_mu;
bool g_attr_set[64];

}  // namespace

// Device address of the error word of the tensor-core kernels on the current device (looked up once per device).
int pd_gemm_error_word(int** out) {
  static int* err_addr[64] = {};
  int dev_now = 0;
  PD_CUDA(cudaGetDevice(&dev_now));
  PD_REQUIRE(dev_now >= 0 && dev_now < 64, "tcgen05 gemm: device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_attr_mu);
  if (err_addr[dev_now] == nullptr) {
    int* e = nullptr;
    PD_CUDA(cudaGetSymbolAddress((void**)&e, g_gemm_error));
    err_addr[dev_now] = e;
  }
  *out = err_addr[dev_now];
  return PD_OK;
}

// Widest N tile that still fills at least half of the SMs; K-major B allows 32-wide tiles, which is what
// keeps a skinny Linear layer (M = batch <= 128) from running on a handful of SMs.
int pd_gemm_pick_block_n(int M, int N, int b_major, int zs) {
  const int sms = pd_num_sms();
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  const int min_bn = b_major ? 64 : 32;
  int bn = N > 128 ? 256 : (N > 64 ? 128 : (N > 32 ? 64 : 32));
  if (bn < min_bn) bn = min_bn;
  // halve only while that at least doubles the busy SMs within one wave: a narrower tile needs more operand
  // rows per FLOP (the TMA row rate bounds short-K tiles), so two thin waves lose against one fat partial wave
  while (bn > min_bn && 2ll * m_tiles * ((N + bn - 1) / bn) * zs <= sms) bn >>= 1;
  return bn;
}

namespace {
int g_pair_mode = 1;     // 1 = CTA pairs where they apply, 0 = single CTAs only (kept for A/B checks of the two tilings)
int g_group_mode = 1;    // 1 = two issuer groups per tile for narrow convolutions, 0 = one
long long* g_stall = nullptr;
}

// A pair of CTAs (256 x 256 tile) is used when the output is at least 256 wide in both directions, the
// problem has one accumulator per tile, and there are enough tiles to give every pair of SMs one.
bool pd_gemm_use_pair(int M, int N, int num_z, int z_group, int split_k) {
  if (!g_pair_mode) return false;
  const int sms = pd_num_sms();
  if (sms < 2 || (sms & 1)) return false;
  if (N < 256 || (N % 256) != 0 || M < 256) return false;
  (void)z_group;
  const long long tiles = (long long)((M + 255) / 256) * (N / 256) * (num_z > 0 ? num_z : 1) * (split_k > 0 ? split_k : 1);
  return tiles >= sms / 2 - sms / 16;     // enough to keep nearly every pair of SMs busy
}

// Chooses between the two tilings of wide problems: 1 (default) lets problems that qualify run on CTA pairs,
// 0 keeps every problem on single CTAs.  Both produce the same sums in the same order.
PD_EXPORT int pd_gemm_set_pair_mode(int mode) {
  g_pair_mode = (mode & 1) ? 1 : 0;
  g_group_mode = (mode & 1) && !(mode & 2) ? 1 : 0;
  return PD_OK;
}

// Diagnostic: with a device buffer of 4 x (number of SMs) int64 the MMA issuer of every CTA adds up, per launch,
// the cycles it waited for operands to land in shared memory, the cycles it waited for a free accumulator, its
// total cycles and its tile count.  NULL switches the counters off (the default).
PD_EXPORT int pd_gemm_set_stall_counters(void* device_buffer) {
  g_stall = (long long*)device_buffer;
  return PD_OK;
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

  int block_n = pd_gemm_pick_block_n(g.M, g.N, g.b_major, g.num_z * g.split_k);
  bool pair = pd_gemm_use_pair(g.M, g.N, g.num_z, g.z_group, g.split_k);
  if (pair) block_n = 256;
  // 3x3 convolutions on a single CTA: 128-wide tiles with the shared tap boxes beat 256-wide ones (the 256-wide
  // tile cannot share the activation box - its stage would not fit - and is then bound by the rate at which
  // one SM pulls operands out of L2) and quantise better into waves of 148 CTAs
  if (g.share_tap_rows && block_n > 128 && !pair) block_n = 128;
  // Narrow convolutions (N = 64 or 128): two 128-row groups per tile, each with its own issuer warp, because one
  // thread cannot issue N <= 128 instructions fast enough to fill the tensor pipe.  N = 64 keeps single CTAs
  // (stage: two activation boxes + three 8 KiB weight tiles, three stages); N = 128 runs on CTA pairs so that each
  // CTA only holds half of the weight tiles and three stages still fit.
  int groups = 1;
  const bool conv9 = g.share_tap_rows && g.num_taps == 9 && !g.a_major && g.num_z == 1 && g.split_k == 1;
  if (g_group_mode && conv9 && !pair) {
    const int sms = pd_num_sms();
    if (g.N == 64 && (long long)((g.M + 255) / 256) >= sms) {
      groups = 2; block_n = 64;
    } else if (g.N == 128 && g_pair_mode && sms >= 2 && !(sms & 1) && (long long)((g.M + 511) / 512) >= sms / 2) {
      groups = 2; block_n = 128; pair = true;
    }
  }
  const int cg = pair ? 2 : 1;
  KParams p;
  memset(&p, 0, sizeof(p));
  p.M = g.M; p.N = g.N; p.block_n = block_n;
  p.cta_n = block_n / cg;
  p.groups = groups;
  p.num_taps = g.num_taps;
  p.kb_per_tap = (g.K + kBlockK - 1) / kBlockK;
  p.split_k = g.split_k;
  if (p.split_k > p.kb_per_tap) p.split_k = p.kb_per_tap;
  p.kb_per_split = (p.kb_per_tap + p.split_k - 1) / p.split_k;
  p.split_k = (p.kb_per_tap + p.kb_per_split - 1) / p.kb_per_split;   // no empty splits
  // z groups: several independent outputs (weight-gradient taps) share one CTA's A tiles
  int acc = g.z_group > 1 ? g.z_group : 1;
  if (acc > 256 / block_n) acc = 256 / block_n;
  if (acc < 1) acc = 1;
  if (acc > g.num_z) acc = g.num_z;
  p.acc_count = acc;
  p.num_z_total = g.num_z;
  p.num_z = (g.num_z + acc - 1) / acc;
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
            ((uint32_t)((kBlockM * cg) >> 4) << 24);
  // shared A boxes for the three taps of a filter row: narrow output tiles only (wide ones are bound by the
  // tensor pipe and want more, smaller stages)
  bool tap3 = g.share_tap_rows && g.num_taps == 9 && !g.a_major && p.cta_n <= 128 && g.num_z == 1 && p.split_k == 1 &&
              p.acc_count == 1;
  for (int r = 0; r < 3 && tap3; ++r) {
    int base = g.a_tap_row[3 * r];
    for (int s3 = 1; s3 < 3; ++s3) base = g.a_tap_row[3 * r + s3] < base ? g.a_tap_row[3 * r + s3] : base;
    p.t3_base[r] = base;
    bool seen[3] = {false, false, false};
    for (int s3 = 0; s3 < 3; ++s3) {
      const int off = g.a_tap_row[3 * r + s3] - base;
      if (off < 0 || off > 2 || seen[off] || g.a_tap_col[3 * r + s3] != 0) { tap3 = false; break; }
      seen[off] = true;
      p.t3_off[3 * r + s3] = off;
    }
  }
  p.tap3 = tap3 ? 1 : 0;
  if (tap3) p.num_taps = 3;
  if (!tap3 && groups > 1) {
    pd_set_error("tcgen05 gemm: internal error, grouped tiles need the shared-tap path");
    return PD_ERR_INVALID;
  }
  const uint32_t stage_bytes = tap3 ? (uint32_t)groups * kA3Bytes + 3u * (uint32_t)p.cta_n * kBlockK * 2
                                    : kABytes + (uint32_t)p.acc_count * (uint32_t)p.cta_n * kBlockK * 2;
  int stages = (int)((200u * 1024u) / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.num_stages = stages;
  {
    const int acc_cols = p.acc_count * block_n;
    int bufs = 512 / (acc_cols * groups);
    p.acc_bufs = bufs > kMaxAccBufs ? kMaxAccBufs : (bufs < 2 ? 2 : bufs);
  }
  p.stall = g_stall;
  {
    int erc = pd_gemm_error_word(&p.err);
    if (erc != PD_OK) return erc;
  }

  CUtensorMap ma, mb;
  int rc = pd_make_map_2d(&ma, g.a, g.a_rows, g.a_cols, g.lda, 64, g.a_major ? kBlockK : (tap3 ? kBox3Rows : kBlockM));
  if (rc != PD_OK) return rc;
  rc = pd_make_map_2d(&mb, g.b, g.b_rows, g.b_cols, g.ldb, 64, g.b_major ? kBlockK : p.cta_n);
  if (rc != PD_OK) return rc;

  const size_t smem = (size_t)stages * stage_bytes + 1024;
  {
    int dev = 0;
    PD_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_attr_mu);
    if (dev >= 0 && dev < 64 && !g_attr_set[dev]) {
      PD_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
      PD_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
      g_attr_set[dev] = true;
    }
  }
  p.m_tiles = (g.M + kBlockM * cg * groups - 1) / (kBlockM * cg * groups);
  p.n_tiles = (g.N + block_n - 1) / block_n;
  make_fast_div((uint32_t)(p.m_tiles * p.n_tiles), p.fd_tiles_mn);
  make_fast_div((uint32_t)p.n_tiles, p.fd_n_tiles);
  make_fast_div((uint32_t)p.num_z, p.fd_num_z);
  make_fast_div((uint32_t)(p.pad_wp > 0 ? p.pad_wp : 1), p.fd_pad_wp);
  make_fast_div((uint32_t)(p.pad_hp > 0 ? p.pad_hp : 1), p.fd_pad_hp);
  const long long total_tiles = (long long)p.m_tiles * p.n_tiles * p.num_z * p.split_k;
  PD_REQUIRE(total_tiles < (1ll << 31), "tcgen05 gemm: too many tiles");
  const int sms = pd_num_sms();
  if (!pair) {
    dim3 grid((unsigned)(total_tiles < sms ? total_tiles : sms), 1, 1);
    gemm_tcgen05_kernel<1><<<grid, kThreads, smem, stream>>>(ma, mb, p);
  } else {
    const long long pairs = sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * (total_tiles < pairs ? total_tiles : pairs)), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    PD_CUDA(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<2>, ma, mb, p));
  }
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
