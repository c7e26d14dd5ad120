// Block-scaled fp8 grouped GEMM with the operand roles exchanged: weights on M, tokens on N.
//
// The kernels in gemm_block.cuh multiply 128-row blocks of sorted tokens, so an expert with
// 260 routed rows pays for 384.  Here the 128 rows of the MMA are weight rows (always full) and
// the tokens are its N extent, which tcgen05.mma accepts in steps of 16: an expert's live rows,
// rounded up to 16, are cut into chunks of at most 224 tokens and nothing else is multiplied.
// moe_sorting's layout is unchanged (every expert still starts at a multiple of 128 slots, live
// rows first); the kernel finds each expert's live count by bisection over sorted_rows.
//
// One tile = (expert, n-block, token chunk):
//   D0[128 x N] = W[slab 0, 128 x K] * X[N x K]^T,   D1[128 x N] = W[slab 1] * X^T
// with slab 0 / 1 = gate rows / up rows of the first GEMM (so SiLU(gate) * up needs no exchange)
// or two consecutive 128-row slabs of the second GEMM's weights.  Both accumulators share the
// token operand in shared memory.  Power-of-two (UE8M0) scales only: tcgen05.mma
// kind::mxf8f6f4.block_scale applies them, the accumulators stay in tensor memory for the whole
// K loop (columns 0.. and 224..), scale columns behind them (448..): per buffer four columns for
// each weight slab (one 128 x 128 block: the same byte on every row) and eight for the tokens.
//
// Warps (384 threads): 0 = TMA producer, 1 = MMA issuer + tensor-memory owner, 2 = scale loader,
// 4..11 = epilogue.  Tensor-memory lane = output channel, column = token, so an epilogue warp's
// store of one column is 32 consecutive channels of one token's row.
//   First GEMM: thread (quadrant q, half h) owns channel 32q + lane and half of the chunk's
//   tokens; it rounds SiLU(g) * u to bf16 in registers, hands the accumulators back, and the
//   128 threads of a half then turn 16 tokens at a time through shared memory so that a warp
//   sees whole 128-channel groups: group maximum, UE8M0 scale, e4m3 bytes, one 128-byte store.
//   Second GEMM: half h owns slab h and all tokens; up to 128 columns are drained to registers
//   before the accumulators are handed back, the rest is stored straight from tensor memory.
#pragma once

#include <cuda_fp8.h>

#include "gemm_block.cuh"

namespace fmoe {

constexpr int kToknThreads = 384;
constexpr int kToknStages = 3;
constexpr int kToknMaxN = 224;                                    // tokens per tile (14 units of 16)
constexpr int kToknWBytes = 2 * kSlabRows * kStageKBytes;         // two weight slabs: 32 KiB
constexpr int kToknStageBytes = kToknWBytes + kToknMaxN * kStageKBytes;   // 60 KiB
constexpr int kToknTableInts = 1028;                              // per-expert tables (<= 1024 experts)
constexpr int kToknMisc = 256 + 3 * kToknTableInts * 4 + 208;     // barriers + three tables, 256-byte multiple
static_assert(kToknMisc % 256 == 0, "keeps the areas behind it aligned");
constexpr int kToknSfSlots = 4;
constexpr int kToknSfSlotBytes = 4 * 512;                         // gate slab, up slab, tokens 0..127, tokens 128..255
constexpr int kToknYStage = 2 * 2 * 16 * 128 * 2;                 // per half, double buffered: 16 tokens x 128 bf16
constexpr int kToknMeta = 2 * kToknMaxN * 8;                      // destination row + weight per token, double buffered
constexpr int kToknSmemBytes = kToknStages * kToknStageBytes + kToknMisc + kToknSfSlots * kToknSfSlotBytes +
                               kToknYStage + kToknMeta + 1024;
static_assert(kToknSmemBytes <= 227 * 1024, "shared memory budget");
constexpr int kToknAcc1Col = kToknMaxN;                           // second accumulator
constexpr int kToknSfCol = 2 * kToknMaxN;                         // 448: scale columns, 16 per buffer
static_assert(kToknSfCol + 2 * 16 <= kTmemCols, "tensor memory budget");

struct ToknTile {
  int expert, n_blk, slot0, ntok;
};

// tile -> (expert, n-block, chunk): experts in order, then n-blocks, chunks fastest, so CTAs
// running side by side share weight slabs through L2.  ccum = cumulative chunks per expert,
// n16 = live rows rounded up to 16, cum = cumulative 128-row blocks (slot of an expert's first row).
__device__ __forceinline__ ToknTile decode_tokn_tile(int tile, const int* ccum, const int* n16, const int* cum,
                                                     int E, int n_blocks) {
  int lo = 1, hi = E;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (ccum[mid] * n_blocks > tile) hi = mid; else lo = mid + 1;
  }
  ToknTile t;
  t.expert = lo - 1;
  const int base_c = ccum[t.expert];
  const int c_e = ccum[t.expert + 1] - base_c;
  const int local = tile - base_c * n_blocks;
  t.n_blk = local / c_e;
  const int chunk = local % c_e;
  const int units = n16[t.expert] >> 4;
  const int per = units / c_e, rem = units % c_e;          // the first `rem` chunks carry one unit more
  const int start = chunk * per + (chunk < rem ? chunk : rem);
  t.slot0 = cum[t.expert] * kBlockM + 16 * start;
  t.ntok = 16 * (per + (chunk < rem ? 1 : 0));
  return t;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int kEpi>
__global__ void __launch_bounds__(kToknThreads, 1)
fmoe_grouped_gemm_tokn_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_t128,
                              const __grid_constant__ CUtensorMap tm_t64, const __grid_constant__ CUtensorMap tm_t32,
                              const __grid_constant__ CUtensorMap tm_t16, const BlockGemmParams bp) {
  static_assert(kEpi == kEpiSiluMul || kEpi == kEpiScaledSlots, "two epilogues");
  const GemmParams& p = bp.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* misc = smem + kToknStages * kToknStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
  uint64_t* empty_bar = full_bar + kToknStages;
  uint64_t* acc_full_bar = empty_bar + kToknStages;
  uint64_t* acc_empty_bar = acc_full_bar + 1;
  uint64_t* sf_full_bar = acc_empty_bar + 1;
  uint64_t* sf_empty_bar = sf_full_bar + kToknSfSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_empty_bar + kToknSfSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* cum_s = reinterpret_cast<int*>(misc + 256);
  int* n16_s = cum_s + kToknTableInts;
  int* ccum_s = n16_s + kToknTableInts;
  uint8_t* sf_ring = misc + kToknMisc;
  uint8_t* y_stage = sf_ring + kToknSfSlots * kToknSfSlotBytes;
  int* meta_rows = reinterpret_cast<int*>(y_stage + kToknYStage);          // [2][kToknMaxN]
  float* meta_w = reinterpret_cast<float*>(meta_rows + 2 * kToknMaxN);     // [2][kToknMaxN]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kUmmaKBytes = 32;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_t128);
    ptx::prefetch_tensormap(&tm_t64);
    ptx::prefetch_tensormap(&tm_t32);
    ptx::prefetch_tensormap(&tm_t16);
    for (int s = 0; s < kToknStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    ptx::mbar_init(ptx::smem_u32(acc_full_bar), 1);
    ptx::mbar_init(ptx::smem_u32(acc_empty_bar), 8);
    for (int s = 0; s < kToknSfSlots; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sf_full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sf_empty_bar[s]), 1);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  // the set-up above needs nothing from the previous kernel; its output is read from here on
  ptx::pdl_wait();
  const int E = p.num_experts;
  for (int i = threadIdx.x; i <= E; i += kToknThreads) cum_s[i] = p.mblk_cum[i];
  __syncthreads();
  // live rows of every expert: first pad slot of its segment (live rows come first)
  for (int e = threadIdx.x; e < E; e += kToknThreads) {
    const int seg0 = cum_s[e] * kBlockM, seg1 = cum_s[e + 1] * kBlockM;
    int lo = seg0, hi = seg1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (p.sorted_rows[mid] < 0) hi = mid; else lo = mid + 1;
    }
    n16_s[e] = ((lo - seg0) + 15) & ~15;
  }
  __syncthreads();
  if (warp == 0) {   // cumulative chunks per expert
    int carry = 0;
    for (int base = 0; base < E; base += 32) {
      const int e = base + lane;
      int v = e < E ? ((n16_s[e] >> 4) + 13) / 14 : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += o;
      }
      if (e < E) ccum_s[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) ccum_s[0] = 0;
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = ccum_s[E] * p.n_blocks;
  const int kb_n = bp.k_blocks;
  const int kg_n = (kb_n + 3) >> 2;        // groups of four K blocks

  if (warp < 4) {
    ptx::setmaxnreg_dec<kBlockThinRegs>();
    if (warp == 0 && lane == 0) {
      // -------------------------------------------------------------- TMA producer
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const ToknTile t = decode_tokn_tile(tile, ccum_s, n16_s, cum_s, E, p.n_blocks);
        const int b_row0 = t.expert * p.b_rows_per_expert + t.n_blk * p.n_stride;
        const int b_row1 = b_row0 + p.second_slab_offset;
        const uint32_t tx = static_cast<uint32_t>(kToknWBytes + t.ntok * kStageKBytes);
        for (int k = 0; k < p.k_iters; ++k) {
          if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&full_bar[stage]);
          const uint32_t sw = ptx::smem_u32(smem + stage * kToknStageBytes);
          ptx::mbar_arrive_expect_tx(full, tx);
          int bx, by0, by1;
          b_coords(p, b_row0, k, 128, bx, by0);
          b_coords(p, b_row1, k, 128, bx, by1);
          ptx::tma_load_2d(sw, &tm_w, full, bx, by0);
          ptx::tma_load_2d(sw + kSlabRows * kStageKBytes, &tm_w, full, bx, by1);
          // the chunk's tokens as at most three boxes (128 + 64 + 32 + 16 rows cover every multiple of 16)
          const int kx = k * 128;
          uint32_t dst = sw + kToknWBytes;
          int r = t.slot0;
          if (t.ntok & 128) { ptx::tma_load_2d(dst, &tm_t128, full, kx, r); dst += 128 * kStageKBytes; r += 128; }
          if (t.ntok & 64) { ptx::tma_load_2d(dst, &tm_t64, full, kx, r); dst += 64 * kStageKBytes; r += 64; }
          if (t.ntok & 32) { ptx::tma_load_2d(dst, &tm_t32, full, kx, r); dst += 32 * kStageKBytes; r += 32; }
          if (t.ntok & 16) { ptx::tma_load_2d(dst, &tm_t16, full, kx, r); }
          if (++stage == kToknStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 0x31);
      ptx::pdl_release();   // all operands requested: the next kernel may begin its set-up
    } else if (warp == 1 && lane == 0) {
      // -------------------------------------------------------------- MMA issuer
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      int sf_slot = 0;
      uint32_t sf_phase = 0;
      int sf_buf = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const ToknTile t = decode_tokn_tile(tile, ccum_s, n16_s, cum_s, E, p.n_blocks);
        if (!ptx::mbar_wait(ptx::smem_u32(acc_empty_bar), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t idesc0 = ptx::make_idesc_block_scaled(kBlockM, static_cast<uint32_t>(t.ntok));
        const uint32_t d0 = tmem_base, d1 = tmem_base + kToknAcc1Col;
        uint32_t sf_w0 = 0, sf_w1 = 0, sf_t = 0;
        for (int k = 0; k < p.k_iters; ++k) {
          if ((k & 3) == 0) {
            if (!ptx::mbar_wait(ptx::smem_u32(&sf_full_bar[sf_slot]), sf_phase, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t src = ptx::smem_u32(sf_ring + sf_slot * kToknSfSlotBytes);
            sf_w0 = tmem_base + static_cast<uint32_t>(kToknSfCol + sf_buf * 16);
            sf_w1 = sf_w0 + 4;
            sf_t = sf_w0 + 8;
            ptx::tmem_cp_32x128b_warpx4(sf_w0, ptx::make_rows16_desc(src));
            ptx::tmem_cp_32x128b_warpx4(sf_w1, ptx::make_rows16_desc(src + 512));
            ptx::tmem_cp_32x128b_warpx4(sf_t, ptx::make_rows16_desc(src + 1024));
            if (t.ntok > 128) ptx::tmem_cp_32x128b_warpx4(sf_t + 4, ptx::make_rows16_desc(src + 1536));
            ptx::umma_commit(ptx::smem_u32(&sf_empty_bar[sf_slot]));   // image may be overwritten once copied
            if (++sf_slot == kToknSfSlots) { sf_slot = 0; sf_phase ^= 1u; }
            sf_buf ^= 1;
          }
          if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sw = ptx::smem_u32(smem + stage * kToknStageBytes);
          const uint64_t dw0 = ptx::make_smem_desc(p.desc_template, sw);
          const uint64_t dw1 = ptx::make_smem_desc(p.desc_template, sw + kSlabRows * kStageKBytes);
          const uint64_t dt = ptx::make_smem_desc(p.desc_template, sw + kToknWBytes);
          const uint32_t idesc = ptx::idesc_with_scale_byte(idesc0, static_cast<uint32_t>(k & 3));
#pragma unroll
          for (int kk = 0; kk < kStageKBytes / kUmmaKBytes; ++kk) {
            const uint64_t adv = static_cast<uint64_t>((kk * kUmmaKBytes) >> 4);
            const uint32_t accumulate = (k | kk) ? 1u : 0u;
            ptx::umma_mxf8_block_scale(d0, dw0 + adv, dt + adv, idesc, sf_w0, sf_t, accumulate);
            ptx::umma_mxf8_block_scale(d1, dw1 + adv, dt + adv, idesc, sf_w1, sf_t, accumulate);
          }
          ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));
          if (++stage == kToknStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        ptx::umma_commit(ptx::smem_u32(acc_full_bar));
        acc_phase ^= 1u;
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 0x32);
    } else if (warp == 2) {
      // -------------------------------------------------------------- scale loader
      int slot = 0;
      uint32_t sphase = 0;
      bool ok = true;
      const uint8_t* a_img = reinterpret_cast<const uint8_t*>(bp.a_scale);   // [a_rows, a_pitch] bytes
      const size_t a_pitch = static_cast<size_t>(scale_pitch(kb_n));
      const long long last_row = bp.a_rows - 1;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const ToknTile t = decode_tokn_tile(tile, ccum_s, n16_s, cum_s, E, p.n_blocks);
        const int b_row0 = t.expert * p.b_rows_per_expert + t.n_blk * p.n_stride;
        // lanes 0..3: K blocks 4g..4g+3 of the first slab's scale block, lanes 4..7: of the second's
        const int w_row = (lane & 4) ? b_row0 + p.second_slab_offset : b_row0;
        const float* sw_l = bp.b_scale + static_cast<size_t>(w_row / 128) * kb_n;
        const int t_groups = (t.ntok + 31) >> 5;       // 32-token groups with live columns
        for (int g = 0; g < kg_n; ++g) {
          // loads first, so their latency overlaps the wait for a free slot
          uint32_t wb = 0;
          {
            const int kb = 4 * g + (lane & 3);
            // a power of two's biased exponent is its UE8M0 byte
            if (lane < 8 && kb < kb_n) wb = ((__float_as_uint(__ldg(sw_l + kb)) >> 23) & 0xffu) << (8 * (lane & 3));
          }
          uint32_t w0 = wb, w1 = __shfl_sync(0xffffffffu, wb, (lane + 4) & 31);   // lane l < 4 receives lane l + 4
          w0 |= __shfl_xor_sync(0xffffffffu, w0, 1);
          w0 |= __shfl_xor_sync(0xffffffffu, w0, 2);
          w1 |= __shfl_xor_sync(0xffffffffu, w1, 1);
          w1 |= __shfl_xor_sync(0xffffffffu, w1, 2);
          w0 = __shfl_sync(0xffffffffu, w0, 0);     // first slab's four bytes
          w1 = __shfl_sync(0xffffffffu, w1, 0);     // second slab's
          // image row `lane` of token group c = the word (K groups 4g..4g+3) of token 32c + lane
          uint32_t tw[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            tw[c] = 0;
            if (c < t_groups) {
              long long row = static_cast<long long>(t.slot0) + 32 * c + lane;
              row = row > last_row ? last_row : row;
              tw[c] = __ldg(reinterpret_cast<const uint32_t*>(a_img + static_cast<size_t>(row) * a_pitch + 4 * g));
            }
          }
          if (!ptx::mbar_wait(ptx::smem_u32(&sf_empty_bar[slot]), sphase ^ 1u, abort_flag)) { ok = false; break; }
          uint4* dst = reinterpret_cast<uint4*>(sf_ring + slot * kToknSfSlotBytes);
          dst[lane] = make_uint4(w0, w0, w0, w0);          // every row of a 128-row slab shares its block's scale
          dst[32 + lane] = make_uint4(w1, w1, w1, w1);
          dst[64 + lane] = make_uint4(tw[0], tw[1], tw[2], tw[3]);
          dst[96 + lane] = make_uint4(tw[4], tw[5], tw[6], tw[7]);
          ptx::fence_proxy_async();      // generic-proxy stores above are read by tcgen05.cp
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sf_full_bar[slot]));
          if (++slot == kToknSfSlots) { slot = 0; sphase ^= 1u; }
        }
      }
      if (!ok && lane == 0) atomicExch(p.status, kStatusGemmTimeout | 0x34);
    }
  } else {
    // ---------------------------------------------------------------- warpgroups 1, 2: epilogue
    ptx::setmaxnreg_inc<kBlockFatRegs>();
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;
    const int et = threadIdx.x - 128;            // 0..255 among the epilogue threads
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    uint32_t acc_phase = 0;
    int par = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const ToknTile t = decode_tokn_tile(tile, ccum_s, n16_s, cum_s, E, p.n_blocks);
      // destination row and routing weight of every token of the chunk, for all epilogue threads
      int* rows_s = meta_rows + par * kToknMaxN;
      float* w_s = meta_w + par * kToknMaxN;
      if (et < t.ntok) {
        rows_s[et] = p.sorted_rows[t.slot0 + et];
        w_s[et] = p.sorted_weights[t.slot0 + et];
      }
      named_bar_sync(3, 256);
      par ^= 1;
      if (!ptx::mbar_wait(ptx::smem_u32(acc_full_bar), acc_phase, abort_flag)) { ok = false; break; }
      acc_phase ^= 1u;
      ptx::tc_fence_after();
      if (kEpi == kEpiSiluMul) {
        // half 0: tokens [0, n0), half 1: [n0, ntok)
        const int n0 = (((t.ntok >> 4) + 1) >> 1) << 4;
        const int cb = half ? n0 : 0;
        const int cn = half ? t.ntok - n0 : n0;
        uint32_t ypk[7][8];                      // SiLU(g) * u rounded to bf16, two tokens per register
#pragma unroll
        for (int j = 0; j < 7; ++j) {
          if (16 * j < cn) {
            uint32_t g[16], u[16];
            ptx::tmem_ld_32x16(t_lane + static_cast<uint32_t>(cb + 16 * j), g);
            ptx::tmem_ld_32x16(t_lane + static_cast<uint32_t>(kToknAcc1Col + cb + 16 * j), u);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const __nv_bfloat162 v2 =
                  __floats2bfloat162_rn(silu(__uint_as_float(g[2 * i])) * __uint_as_float(u[2 * i]),
                                        silu(__uint_as_float(g[2 * i + 1])) * __uint_as_float(u[2 * i + 1]));
              ypk[j][i] = *reinterpret_cast<const uint32_t*>(&v2);
            }
          }
        }
        // both accumulators are in registers: the next tile may overwrite tensor memory
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(acc_empty_bar));
        // 16 tokens at a time through shared memory: [token][channel] bf16, then one warp per token group
        uint16_t* ys = reinterpret_cast<uint16_t*>(y_stage) + half * (2 * 16 * 128);
        const int ch = quad * 32 + lane;
        const int groups = p.ld_out >> 7;
        uint8_t* qbase = reinterpret_cast<uint8_t*>(p.out) + t.n_blk * kSlabRows + 4 * lane;
        uint8_t* sbase = reinterpret_cast<uint8_t*>(bp.out_scale) + t.n_blk;
        const size_t spitch = static_cast<size_t>(scale_pitch(groups));
#pragma unroll
        for (int j = 0; j < 7; ++j) {
          if (16 * j < cn) {
            uint16_t* buf = ys + (j & 1) * (16 * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              buf[(2 * i) * 128 + ch] = static_cast<uint16_t>(ypk[j][i] & 0xffffu);
              buf[(2 * i + 1) * 128 + ch] = static_cast<uint16_t>(ypk[j][i] >> 16);
            }
            named_bar_sync(1 + half, 128);
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
              const int tok = 4 * quad + tt;
              const int c = cb + 16 * j + tok;
              const uint2 raw = *reinterpret_cast<const uint2*>(buf + tok * 128 + 4 * lane);
              const float f0 = __uint_as_float(raw.x << 16), f1 = __uint_as_float(raw.x & 0xffff0000u);
              const float f2 = __uint_as_float(raw.y << 16), f3 = __uint_as_float(raw.y & 0xffff0000u);
              float amax = fmaxf(fmaxf(fabsf(f0), fabsf(f1)), fmaxf(fabsf(f2), fabsf(f3)));
#pragma unroll
              for (int d = 16; d >= 1; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
              uint32_t sbyte;
              const float sc = group_scale<true>(amax, sbyte);
              const float inv = 1.0f / sc;
              const uint32_t word =
                  static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f0 * inv, f1 * inv), __NV_SATFINITE, __NV_E4M3)) |
                  (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(f2 * inv, f3 * inv), __NV_SATFINITE, __NV_E4M3)) << 16);
              const int slot = t.slot0 + c;
              if (rows_s[c] >= 0 && FMOE_ROW_OK(p, slot)) {
                *reinterpret_cast<uint32_t*>(qbase + static_cast<size_t>(slot) * p.ld_out) = word;
                if (lane == 0) sbase[static_cast<size_t>(slot) * spitch] = static_cast<uint8_t>(sbyte);
              }
            }
          }
        }
      } else {
        // half h owns slab h: output channel n_blk * 256 + 128 h + 32 q + lane, every token of the chunk
        const uint32_t t_acc = t_lane + static_cast<uint32_t>(half * kToknAcc1Col);
        const int chan = t.n_blk * kTileN + half * kSlabRows + quad * 32 + lane;
        auto store16 = [&](int c0, const uint32_t (&v)[16]) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int row = rows_s[c0 + i];
            if (row >= 0 && FMOE_ROW_OK(p, row)) {
              const float val = w_s[c0 + i] * __uint_as_float(v[i]);
              if (p.out_bf16) {
                __nv_bfloat16* drow = p.row_ptrs ? reinterpret_cast<__nv_bfloat16*>(p.row_ptrs[row])
                                                 : reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(row) * p.ld_out;
                drow[chan] = __float2bfloat16_rn(val);
              } else {
                reinterpret_cast<float*>(p.out)[static_cast<size_t>(row) * p.ld_out + chan] = val;
              }
            }
          }
        };
        uint32_t v[8][16];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (16 * j < t.ntok) ptx::tmem_ld_32x16(t_acc + static_cast<uint32_t>(16 * j), v[j]);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 8; j < 14; ++j) {           // columns beyond 128 go out while tensor memory is still held
          if (16 * j < t.ntok) {
            uint32_t x[16];
            ptx::tmem_ld_32x16(t_acc + static_cast<uint32_t>(16 * j), x);
            ptx::tmem_ld_wait();
            store16(16 * j, x);
          }
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(acc_empty_bar));
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (16 * j < t.ntok) store16(16 * j, v[j]);
      }
    }
    if (!ok && threadIdx.x == 128) atomicExch(p.status, kStatusGemmTimeout | 0x33);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (kEpi == kEpiScaledSlots) grid_done_signal(p);
}

}  // namespace fmoe
