// Block-scaled fp8 grouped GEMMs: 1x128 activation groups x 128x128 weight blocks, i.e. a new
// pair of scales every 128 elements of K, which is exactly one pipeline stage of e4m3.
//
// Two flavours of one kernel (template parameter kHw):
//
//   kHw = false, f32 scales.  The MMAs of one stage write a *partial* product into one of two
//   256-column TMEM buffers (no accumulation across stages) and eight epilogue warps promote it:
//   acc += partial * (s_act[row, kb] * s_w[nblock, kb]), running sums in registers.
//
//   kHw = true, power-of-two (UE8M0) scales.  tcgen05.mma kind::mxf8f6f4.block_scale applies the
//   scales inside the tensor core, so one 256-column accumulator stays in tensor memory for the
//   whole K loop, as in the unscaled kernels.  A scale column of tensor memory holds four bytes
//   per row; they are filled with the scales of four consecutive K blocks and every stage selects
//   its byte through the instruction descriptor, so scales are copied to tensor memory (tcgen05.cp)
//   once per four stages.  Warp 2 stages them in shared memory as the 32 x 16-byte image that copy
//   reads: the activation scales are row-major bytes, four K groups to a word, so an image row is
//   four word loads; the weight scales are turned from f32 powers of two into exponent bytes and
//   replicated over the slab's 128 rows on the fly.
//   When the accumulator is complete the eight epilogue warps drain it into registers, hand the
//   tensor memory back at once and run their epilogue while the next tile is multiplied.
//
// Epilogue (both flavours): thread (quadrant q, half h) owns row 32q+lane and, for the first GEMM,
// gate columns [64h, 64h+64) and the matching up columns, so SiLU(gate)*up needs no exchange; the
// 128 columns of a tile are one 1x128 quantisation group of the intermediate, so the two halves
// exchange their maxima through shared memory and the tile is stored as e4m3 with its scale -- the
// intermediate never exists as bf16 in memory (it is rounded to bf16 in registers first, which is
// the rounding point of the arithmetic contract).  For the second GEMM the thread owns output
// channels [128h, 128h+128), one weight-scale block.
#pragma once

#include <cuda_fp8.h>

#include "gemm.cuh"
#include "scales.cuh"

namespace fmoe {

constexpr int kBlockGemmThreads = 384;   // warpgroup 0: producer, MMA, scale loader; warpgroups 1, 2: epilogue
constexpr int kBlockStages = 4;
constexpr int kScaleAhead = 4;           // K blocks between the load of an f32 scale and its use
// setmaxnreg only redistributes what the CTA was given at launch (384 threads x 168 registers):
// the per-role counts must add up to no more than that, or setmaxnreg.inc never returns.
constexpr int kBlockThinRegs = 40;       // registers per thread kept by warpgroup 0
constexpr int kBlockFatRegs = 232;       // registers per thread taken by the epilogue warpgroups
static_assert(128 * kBlockThinRegs + 256 * kBlockFatRegs <= kBlockGemmThreads * 168, "register budget");
constexpr int kBlockMisc = 4608;                     // barriers (256 B) + block table (<= 1025 ints)
constexpr int kBlockEpiStage = 8 * 32 * 20 * 4;      // per-warp transpose areas of the eight epilogue warps
constexpr int kSfSlots = 4;                          // shared-memory ring of scale images (hardware-scaled flavour)
constexpr int kSfSlotBytes = 512 + 2 * 512;          // activation rows + two weight slabs
constexpr int kBlockXchg = 2 * 2 * 128 * 4;          // group maxima of the two halves, double buffered
constexpr int kBlockSmemBytes = kBlockStages * kStageBytes + kBlockMisc + kBlockEpiStage +
                                kSfSlots * kSfSlotBytes + kBlockXchg + 1024;
static_assert(kBlockSmemBytes <= 227 * 1024, "shared memory budget");
constexpr int kSfTmemCol = 256;          // scale columns start behind the accumulator; 16 columns per buffer

struct BlockGemmParams {
  GemmParams g;                 // a_scale / b_scale of g are unused here
  const void* a_scale;          // f32 [cap, k_blocks], or UE8M0 bytes [cap, scale_pitch(k_blocks)] (kHw)
  const float* b_scale;         // [E * b_rows_per_expert / 128, k_blocks]
  int k_blocks;                 // K / 128 (== g.k_iters)
  int64_t a_rows;               // rows of the activation matrix and of a_scale
  void* out_scale;              // first GEMM: scales of the quantised intermediate, f32 [cap, ld_out/128]
                                // or UE8M0 bytes [cap, scale_pitch(ld_out/128)] (kHw); `g.out` then receives e4m3
};

// kNT: accumulator columns of one tile.  256 in general.  224 is the double-buffered form of the
// hardware-scaled second GEMM: two 224-column accumulators and the scale buffers fit the 512
// columns of tensor memory (2 * 224 + 2 * 16), so the drain of tile i overlaps the MMAs of tile
// i+1; it needs an output width that is a multiple of 224 (7168 = 32 * 224) and row-major weights.
template <int kEpi, bool kHw, int kNT = kTileN>
__global__ void __launch_bounds__(kBlockGemmThreads, 1)
fmoe_grouped_gemm_block_kernel(const __grid_constant__ CUtensorMap tm_a,
                               const __grid_constant__ CUtensorMap tm_b, const BlockGemmParams bp) {
  const GemmParams& p = bp.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* misc = smem + kBlockStages * kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);
  uint64_t* empty_bar = full_bar + kBlockStages;
  uint64_t* part_full_bar = empty_bar + kBlockStages;                // [2] partial / accumulator ready
  uint64_t* part_empty_bar = part_full_bar + 2;                      // [2] partial / accumulator consumed
  uint64_t* sf_full_bar = part_empty_bar + 2;                        // [kSfSlots] scale image staged
  uint64_t* sf_empty_bar = sf_full_bar + kSfSlots;                   // [kSfSlots] scale image copied
  uint64_t* xchg_bar = sf_empty_bar + kSfSlots;                      // [4] group-maximum exchange per quadrant
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xchg_bar + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* cum_s = reinterpret_cast<int*>(misc + 256);
  uint8_t* epi_stage = misc + kBlockMisc;
  uint8_t* sf_ring = epi_stage + kBlockEpiStage;
  float* xchg = reinterpret_cast<float*>(sf_ring + kSfSlots * kSfSlotBytes);   // [2][2][128]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kUmmaKBytes = 32;
  static_assert(kNT == kTileN || (kNT == 224 && kHw && kEpi == kEpiScaledSlots), "224-column tiles: hardware-scaled second GEMM only");
  constexpr int kSlab = kNT / 2;                       // rows of one B slab
  constexpr int kAccBufs = kNT == kTileN ? 1 : 2;      // accumulators in tensor memory (hardware-scaled flavour)
  constexpr int kSfCol = kAccBufs * kNT;               // scale columns start behind the accumulators
  constexpr int kTxBytes = kABytes + kNT * kStageKBytes;

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_a);
    ptx::prefetch_tensormap(&tm_b);
    for (int s = 0; s < kBlockStages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(&part_full_bar[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&part_empty_bar[b]), 8);
    }
    for (int s = 0; s < kSfSlots; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sf_full_bar[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sf_empty_bar[s]), 1);
    }
    for (int q = 0; q < 4; ++q) ptx::mbar_init(ptx::smem_u32(&xchg_bar[q]), 2);
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
  for (int i = threadIdx.x; i <= p.num_experts; i += kBlockGemmThreads) cum_s[i] = p.mblk_cum[i];
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = cum_s[p.num_experts] * p.n_blocks;
  const int kb_n = bp.k_blocks;
  const int kg_n = (kb_n + 3) >> 2;        // groups of four K blocks

  if (warp < 4) {
    // -------------------------------------------------------------- warpgroup 0: data movement and MMA issue
    ptx::setmaxnreg_dec<kBlockThinRegs>();
    if (warp == 0 && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord tc = decode_tile(tile, cum_s, p.num_experts, p.n_blocks);
        const int a_row = tc.m_blk * kBlockM;
        const int b_row0 = tc.expert * p.b_rows_per_expert + tc.n_blk * p.n_stride;
        const int b_row1 = b_row0 + p.second_slab_offset;
        for (int k = 0; k < p.k_iters; ++k) {
          if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&full_bar[stage]);
          const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kABytes;
          if (FMOE_DBG(p, 32u)) {     // timing experiment: no operand traffic at all
            ptx::mbar_arrive(full);
            if (++stage == kBlockStages) { stage = 0; phase ^= 1u; }
            continue;
          }
          ptx::mbar_arrive_expect_tx(full, kTxBytes);
          const int kx = k * 128;
          int bx, by0, by1;
          b_coords(p, b_row0, k, 128, bx, by0);
          b_coords(p, b_row1, k, 128, bx, by1);
          ptx::tma_load_2d(sa, &tm_a, full, kx, a_row);
          ptx::tma_load_2d(sb, &tm_b, full, bx, by0);
          ptx::tma_load_2d(sb + kSlab * kStageKBytes, &tm_b, full, bx, by1);
          if (++stage == kBlockStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 0x21);
      ptx::pdl_release();   // all operands requested: the next kernel may begin its set-up
    } else if (warp == 1 && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      if (kHw) {
        // accumulator(s) stay in tensor memory; scales copied there once per four stages
        int acc = 0;
        uint32_t acc_phase = 0;
        int sf_slot = 0;
        uint32_t sf_phase = 0;
        int sf_buf = 0;
        const uint32_t idesc0 = ptx::make_idesc_block_scaled(kBlockM, kNT);
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
          if (!ptx::mbar_wait(ptx::smem_u32(&part_empty_bar[acc]), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kNT);
          uint32_t sfa_t = 0, sfb_t = 0;
          for (int k = 0; k < p.k_iters; ++k) {
            if ((k & 3) == 0) {
              if (!ptx::mbar_wait(ptx::smem_u32(&sf_full_bar[sf_slot]), sf_phase, abort_flag)) { ok = false; break; }
              ptx::tc_fence_after();
              const uint32_t src = ptx::smem_u32(sf_ring + sf_slot * kSfSlotBytes);
              sfa_t = tmem_base + static_cast<uint32_t>(kSfCol + sf_buf * 16);
              sfb_t = sfa_t + 4;
              ptx::tmem_cp_32x128b_warpx4(sfa_t, ptx::make_rows16_desc(src));
              ptx::tmem_cp_32x128b_warpx4(sfb_t, ptx::make_rows16_desc(src + 512));
              ptx::tmem_cp_32x128b_warpx4(sfb_t + 4, ptx::make_rows16_desc(src + 1024));
              ptx::umma_commit(ptx::smem_u32(&sf_empty_bar[sf_slot]));   // image may be overwritten once copied
              if (++sf_slot == kSfSlots) { sf_slot = 0; sf_phase ^= 1u; }
              sf_buf ^= 1;
            }
            if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytes);
            const uint64_t da = ptx::make_smem_desc(p.desc_template, sa);
            const uint64_t db = ptx::make_smem_desc(p.desc_template, sa + kABytes);
            const uint32_t idesc = ptx::idesc_with_scale_byte(idesc0, static_cast<uint32_t>(k & 3));
#pragma unroll
            for (int kk = 0; kk < kStageKBytes / kUmmaKBytes; ++kk) {
              const uint64_t adv = static_cast<uint64_t>((kk * kUmmaKBytes) >> 4);
              if (!FMOE_DBG(p, 2u))
                ptx::umma_mxf8_block_scale(d_tmem, da + adv, db + adv, idesc, sfa_t, sfb_t, (k | kk) ? 1u : 0u);
            }
            ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));
            if (++stage == kBlockStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          ptx::umma_commit(ptx::smem_u32(&part_full_bar[acc]));
          if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
        }
      } else {
        int buf = 0;
        uint32_t buf_phase = 0;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
          for (int k = 0; k < p.k_iters; ++k) {
            if (!ptx::mbar_wait(ptx::smem_u32(&part_empty_bar[buf]), buf_phase ^ 1u, abort_flag) ||
                !ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * kTileN);
            const uint32_t sa = ptx::smem_u32(smem + stage * kStageBytes);
            const uint64_t da = ptx::make_smem_desc(p.desc_template, sa);
            const uint64_t db = ptx::make_smem_desc(p.desc_template, sa + kABytes);
#pragma unroll
            for (int kk = 0; kk < kStageKBytes / kUmmaKBytes; ++kk) {
              const uint64_t adv = static_cast<uint64_t>((kk * kUmmaKBytes) >> 4);
              if (!FMOE_DBG(p, 2u))
                ptx::umma_f8(d_tmem, da + adv, db + adv, p.idesc, kk ? 1u : 0u);   // fresh partial per stage
            }
            ptx::umma_commit(ptx::smem_u32(&empty_bar[stage]));
            ptx::umma_commit(ptx::smem_u32(&part_full_bar[buf]));
            if (++stage == kBlockStages) { stage = 0; phase ^= 1u; }
            if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
          }
        }
      }
      if (!ok) atomicExch(p.status, kStatusGemmTimeout | 0x22);
    } else if (kHw && warp == 2) {
      // ------------------------------------------------------------ scale loader (hardware-scaled flavour)
      int slot = 0;
      uint32_t sphase = 0;
      bool ok = true;
      const uint8_t* a_img = reinterpret_cast<const uint8_t*>(bp.a_scale);   // [rows, a_pitch] bytes
      const size_t a_pitch = static_cast<size_t>(scale_pitch(kb_n));
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const TileCoord tc = decode_tile(tile, cum_s, p.num_experts, p.n_blocks);
        const int b_row0 = tc.expert * p.b_rows_per_expert + tc.n_blk * p.n_stride;
        // lane c < 8 serves the 32-row group c of the B tile: rows below kSlab belong to the first
        // slab, the others to the second; a group never straddles a 128-row scale block
        const int grow = 32 * (lane & 7);
        const int g_row = grow < kSlab ? b_row0 + grow : b_row0 + p.second_slab_offset + (grow - kSlab);
        const float* sb_l = bp.b_scale + static_cast<size_t>(g_row / 128) * kb_n;
        const bool g_live = grow < kNT;
        for (int g = 0; g < kg_n; ++g) {
          // loads first, so their latency overlaps the wait for a free slot
          // image row `lane` = the four-byte words (K groups 4g..4g+3) of rows lane, 32+lane, 64+lane, 96+lane
          const uint8_t* arow = a_img + (static_cast<size_t>(tc.m_blk) * kBlockM + lane) * a_pitch + 4 * g;
          uint4 av;
          av.x = __ldg(reinterpret_cast<const uint32_t*>(arow));
          av.y = __ldg(reinterpret_cast<const uint32_t*>(arow + 32 * a_pitch));
          av.z = __ldg(reinterpret_cast<const uint32_t*>(arow + 64 * a_pitch));
          av.w = __ldg(reinterpret_cast<const uint32_t*>(arow + 96 * a_pitch));
          uint32_t wl = 0;
          if (g_live) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int kb = 4 * g + j;
              // a power of two's biased exponent is its UE8M0 byte
              if (kb < kb_n) wl |= ((__float_as_uint(__ldg(sb_l + kb)) >> 23) & 0xffu) << (8 * j);
            }
          }
          uint32_t w[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) w[c] = __shfl_sync(0xffffffffu, wl, c);
          if (!ptx::mbar_wait(ptx::smem_u32(&sf_empty_bar[slot]), sphase ^ 1u, abort_flag)) { ok = false; break; }
          uint4* dst = reinterpret_cast<uint4*>(sf_ring + slot * kSfSlotBytes);
          dst[lane] = av;
          dst[32 + lane] = make_uint4(w[0], w[1], w[2], w[3]);     // every row of a 32-row group shares its scale
          dst[64 + lane] = make_uint4(w[4], w[5], w[6], w[7]);
          ptx::fence_proxy_async();      // generic-proxy stores above are read by tcgen05.cp
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sf_full_bar[slot]));
          if (++slot == kSfSlots) { slot = 0; sphase ^= 1u; }
        }
      }
      if (!ok && lane == 0) atomicExch(p.status, kStatusGemmTimeout | 0x24);
    }
  } else {
    // -------------------------------------------------------------- warpgroups 1, 2: promotion / drain + epilogue
    ptx::setmaxnreg_inc<kBlockFatRegs>();
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;
    int buf = 0;
    uint32_t buf_phase = 0;
    uint32_t xphase = 0;
    int xbuf = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const TileCoord tc = decode_tile(tile, cum_s, p.num_experts, p.n_blocks);
      const int slot = tc.m_blk * kBlockM + quad * 32 + lane;
      const int b_row0 = tc.expert * p.b_rows_per_expert + tc.n_blk * p.n_stride;
      uint64_t acc[64];          // 128 f32 values, two per register pair
      // TMEM columns of this thread's two 64-column runs
      const int col0 = (kEpi == kEpiSiluMul) ? half * 64 : half * 128;
      const int col1 = (kEpi == kEpiSiluMul) ? kSlabRows + half * 64 : half * 128 + 64;
      if (kHw) {
        if (!ptx::mbar_wait(ptx::smem_u32(&part_full_bar[buf]), buf_phase, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        // A warp whose 32 rows are all padding has nothing to store: it hands the accumulator
        // back without reading it.  Its partner warp of the other column half sees the same rows
        // and does the same, so the group-maximum exchange stays in step.
        if (__ballot_sync(0xffffffffu, p.sorted_rows[slot] >= 0) == 0u) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&part_empty_bar[buf]));
          if (++buf == kAccBufs) { buf = 0; buf_phase ^= 1u; }
          continue;
        }
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(buf * kNT);
        if (kNT == kTileN) {
#pragma unroll
          for (int rnd = 0; rnd < 2; ++rnd) {
            uint32_t v[2][32];
            const int cbase = rnd == 0 ? col0 : col1;
            ptx::tmem_ld_32x32(t_row + cbase, v[0]);
            ptx::tmem_ld_32x32(t_row + cbase + 32, v[1]);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int j = 0; j < 16; ++j)
                acc[rnd * 32 + c * 16 + j] = ptx::pack2(__uint_as_float(v[c][2 * j]), __uint_as_float(v[c][2 * j + 1]));
          }
        } else {
          // 112 columns per thread: 32 + 32 + 32 + 16
          const int cb = half * (kNT / 2);
          uint32_t v[2][32];
          ptx::tmem_ld_32x32(t_row + cb, v[0]);
          ptx::tmem_ld_32x32(t_row + cb + 32, v[1]);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int j = 0; j < 16; ++j)
              acc[c * 16 + j] = ptx::pack2(__uint_as_float(v[c][2 * j]), __uint_as_float(v[c][2 * j + 1]));
          uint32_t t16[16];
          ptx::tmem_ld_32x32(t_row + cb + 64, v[0]);
          ptx::tmem_ld_32x16(t_row + cb + 96, t16);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[32 + j] = ptx::pack2(__uint_as_float(v[0][2 * j]), __uint_as_float(v[0][2 * j + 1]));
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[48 + j] = ptx::pack2(__uint_as_float(t16[2 * j]), __uint_as_float(t16[2 * j + 1]));
        }
        // the accumulator is in registers: a later tile may overwrite this part of tensor memory
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&part_empty_bar[buf]));
        if (++buf == kAccBufs) { buf = 0; buf_phase ^= 1u; }
      } else {
        const float* a_scale_f = reinterpret_cast<const float*>(bp.a_scale);
        const float* sa_row = a_scale_f + static_cast<size_t>(slot) * kb_n;
        const float* sb0;
        const float* sb1;
        if (kEpi == kEpiSiluMul) {
          sb0 = bp.b_scale + static_cast<size_t>(b_row0 / 128) * kb_n;                          // gate slab
          sb1 = bp.b_scale + static_cast<size_t>((b_row0 + p.second_slab_offset) / 128) * kb_n; // up slab
        } else {
          sb0 = bp.b_scale + static_cast<size_t>(b_row0 / 128 + half) * kb_n;
          sb1 = sb0;
        }
#pragma unroll
        for (int j = 0; j < 64; ++j) acc[j] = 0ull;
        // Scales are fetched kScaleAhead K blocks before they are used: the per-row loads miss
        // the small L1 that is left beside the shared memory, and an L2 round trip takes longer
        // than one stage.  The row's activation scales come four at a time (one 16-byte load per
        // four stages) when the rows of the scale matrix are whole, aligned float4s.
        static_assert(kScaleAhead == 4, "the vector path loads one float4 per block of stages");
        const bool vec4 = (kb_n & 3) == 0 && (reinterpret_cast<uintptr_t>(a_scale_f) & 15) == 0;
        float q_act[kScaleAhead], n_act[kScaleAhead], q_b0[kScaleAhead], q_b1[kScaleAhead];
        if (vec4) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(sa_row));
          q_act[0] = t.x; q_act[1] = t.y; q_act[2] = t.z; q_act[3] = t.w;
        }
#pragma unroll
        for (int u = 0; u < kScaleAhead; ++u) {
          n_act[u] = 0.f;
          if (u < p.k_iters) {
            if (!vec4) q_act[u] = __ldg(sa_row + u);
            q_b0[u] = __ldg(sb0 + u);
            q_b1[u] = kEpi == kEpiSiluMul ? __ldg(sb1 + u) : q_b0[u];
          }
        }
        for (int k0 = 0; ok && k0 < p.k_iters; k0 += kScaleAhead) {
          if (vec4 && k0 + kScaleAhead < p.k_iters) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(sa_row + k0 + kScaleAhead));
            n_act[0] = t.x; n_act[1] = t.y; n_act[2] = t.z; n_act[3] = t.w;
          }
#pragma unroll
          for (int u = 0; u < kScaleAhead; ++u) {
            const int k = k0 + u;
            if (k >= p.k_iters) break;
            const float sc0 = q_act[u] * q_b0[u], sc1 = q_act[u] * q_b1[u];
            const uint64_t sc0_2 = ptx::pack2(sc0, sc0), sc1_2 = ptx::pack2(sc1, sc1);
            if (k + kScaleAhead < p.k_iters) {
              if (!vec4) q_act[u] = __ldg(sa_row + k + kScaleAhead);
              q_b0[u] = __ldg(sb0 + k + kScaleAhead);
              q_b1[u] = kEpi == kEpiSiluMul ? __ldg(sb1 + k + kScaleAhead) : q_b0[u];
            }
            if (!ptx::mbar_wait(ptx::smem_u32(&part_full_bar[buf]), buf_phase, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                                   static_cast<uint32_t>(buf * kTileN);
            uint32_t v[2][32];
            // The loop is register-tight (232 per thread: 128 sums, 64 loaded values, the scales in
            // flight).  Its phases -- two loads, FMAs, two loads, FMAs -- stay separate basic
            // blocks behind conditions that are always true but not provable (k_blocks > 0, n_blocks > 0): without
            // them the compiler overlaps the phases' live ranges and spills inside the loop (208
            // bytes of spill stores in the second GEMM's instance, 2.7 ms instead of 2.1 ms).
            const bool dbg_no_ld = FMOE_DBG(p, 4u) || bp.k_blocks <= 0, dbg_no_fma = FMOE_DBG(p, 1u) || p.n_blocks <= 0;
            if (!dbg_no_ld) {
              ptx::tmem_ld_32x32(t_row + col0, v[0]);
              ptx::tmem_ld_32x32(t_row + col0 + 32, v[1]);
              ptx::tmem_ld_wait();
            }
            if (!dbg_no_fma) {
#pragma unroll
              for (int j = 0; j < 16; ++j) ptx::fma2(acc[j], v[0][2 * j], v[0][2 * j + 1], sc0_2);
            }
            if (!dbg_no_ld) ptx::tmem_ld_32x32(t_row + col1, v[0]);
            if (!dbg_no_fma) {
#pragma unroll
              for (int j = 0; j < 16; ++j) ptx::fma2(acc[16 + j], v[1][2 * j], v[1][2 * j + 1], sc0_2);
            }
            if (!dbg_no_ld) {
              ptx::tmem_ld_32x32(t_row + col1 + 32, v[1]);
              ptx::tmem_ld_wait();
            }
            // all four loads have landed: the buffer can be overwritten while the last FMAs run
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&part_empty_bar[buf]));
            if (!dbg_no_fma) {
#pragma unroll
              for (int j = 0; j < 16; ++j) ptx::fma2(acc[32 + j], v[0][2 * j], v[0][2 * j + 1], sc1_2);
#pragma unroll
              for (int j = 0; j < 16; ++j) ptx::fma2(acc[48 + j], v[1][2 * j], v[1][2 * j + 1], sc1_2);
            }
            if (++buf == 2) { buf = 0; buf_phase ^= 1u; }
          }
          if (vec4) {
#pragma unroll
            for (int u = 0; u < kScaleAhead; ++u) q_act[u] = n_act[u];
          }
        }
        if (!ok) break;
      }
      if (FMOE_DBG(p, 16u)) continue;
      // ------------------------------------------------------------ fused epilogue on the 128 values in registers
      // Stores go through a per-warp transpose (32 rows x 16 words at a time) so each store
      // instruction writes 64-byte row segments instead of 16 bytes to 32 different rows.
      uint32_t* stage = reinterpret_cast<uint32_t*>(epi_stage) + (warp - 4) * (32 * 20);
      const int row = p.sorted_rows[slot];
      const int slot0 = slot - lane;
      const int row_in_blk = quad * 32 + lane;
      if (kEpi == kEpiSiluMul) {
        // pairs 0..31: gate, 32..63: up, columns n_blk*128 + half*64 ..  The intermediate is
        // rounded to bf16 (the contract's rounding point) and kept as bf16 pairs.
        uint32_t yb[32];
        __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float g0, g1, u0, u1;
          ptx::unpack2(acc[j], g0, g1);
          ptx::unpack2(acc[32 + j], u0, u1);
          const __nv_bfloat162 v2 = __floats2bfloat162_rn(silu(g0) * u0, silu(g1) * u1);
          amax2 = __hmax2(amax2, __habs2(v2));
          yb[j] = *reinterpret_cast<const uint32_t*>(&v2);
        }
        float amax = fmaxf(__low2float(amax2), __high2float(amax2));
        // the other half of this row's 128-column group lives in the partner warp
        float* xrow = xchg + xbuf * 256;
        xrow[half * 128 + row_in_blk] = amax;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&xchg_bar[quad]));
        if (!ptx::mbar_wait(ptx::smem_u32(&xchg_bar[quad]), xphase, abort_flag)) { ok = false; break; }
        amax = fmaxf(amax, xrow[(half ^ 1) * 128 + row_in_blk]);
        xphase ^= 1u;
        xbuf ^= 1;
        uint32_t sbyte;
        const float sc = group_scale<kHw>(amax, sbyte);
        const float inv = 1.0f / sc;
        if (half == 0 && row >= 0 && FMOE_ROW_OK(p, slot)) {
          const int groups = p.ld_out >> 7;
          if (kHw)
            reinterpret_cast<uint8_t*>(bp.out_scale)[static_cast<size_t>(slot) * scale_pitch(groups) + tc.n_blk] =
                static_cast<uint8_t>(sbyte);
          else
            reinterpret_cast<float*>(bp.out_scale)[static_cast<size_t>(slot) * groups + tc.n_blk] = sc;
        }
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          uint32_t word = 0;
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            const uint32_t bits = yb[2 * j + h2];
            const float2 f = make_float2(__uint_as_float(bits << 16) * inv, __uint_as_float(bits & 0xffff0000u) * inv);
            word |= static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3)) << (16 * h2);
          }
          w[j] = word;
        }
        uint8_t* qbase = reinterpret_cast<uint8_t*>(p.out) + tc.n_blk * kSlabRows + half * 64;
        __syncwarp();
#pragma unroll
        for (int q = 0; q < 4; ++q)
          reinterpret_cast<uint4*>(stage + lane * 20)[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int r = it * 8 + (lane >> 2);
          const int seg = lane & 3;
          const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 20 + seg * 4);
          if (__shfl_sync(0xffffffffu, row, r) >= 0 && FMOE_ROW_OK(p, slot0 + r))
            *reinterpret_cast<uint4*>(qbase + static_cast<size_t>(slot0 + r) * p.ld_out + seg * 16) = val;
        }
      } else if (kEpi == kEpiScaledSlots) {
        const float wt = p.sorted_weights[slot];
        constexpr int kOwn = kNT / 2;                 // output channels of this thread: acc[0 .. kOwn/2)
        const int col_base = tc.n_blk * kNT + half * kOwn;
        if (p.out_bf16) {
          __nv_bfloat16* hbase = reinterpret_cast<__nv_bfloat16*>(p.out) + col_base;
#pragma unroll
          for (int ch = 0; ch < kOwn / 16; ++ch) {     // 16 columns (8 bf16 pairs) per chunk
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float a0, a1;
              ptx::unpack2(acc[ch * 8 + j], a0, a1);
              const __nv_bfloat162 v2 = __floats2bfloat162_rn(wt * a0, wt * a1);
              w[j] = *reinterpret_cast<const uint32_t*>(&v2);
            }
            __syncwarp();
            reinterpret_cast<uint4*>(stage + lane * 20)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(stage + lane * 20)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 2; ++it) {           // 2 lanes per row, 16 rows per store instruction
              const int r = it * 16 + (lane >> 1);
              const int seg = lane & 1;
              const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 20 + seg * 4);
              const int row_r = __shfl_sync(0xffffffffu, row, r);
              if (row_r >= 0 && FMOE_ROW_OK(p, row_r)) {
                __nv_bfloat16* drow = p.row_ptrs ? reinterpret_cast<__nv_bfloat16*>(p.row_ptrs[row_r]) + col_base
                                                 : hbase + static_cast<size_t>(row_r) * p.ld_out;
                *reinterpret_cast<uint4*>(drow + ch * 16 + seg * 8) = val;
              }
            }
          }
        } else {
          float* obase = reinterpret_cast<float*>(p.out) + col_base;
#pragma unroll
          for (int ch = 0; ch < kOwn / 16; ++ch) {     // 16 columns per chunk
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float a0, a1, a2, a3;
              ptx::unpack2(acc[ch * 8 + 2 * q], a0, a1);
              ptx::unpack2(acc[ch * 8 + 2 * q + 1], a2, a3);
              reinterpret_cast<float4*>(stage + lane * 20)[q] = make_float4(wt * a0, wt * a1, wt * a2, wt * a3);
            }
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 4; ++it) {
              const int r = it * 8 + (lane >> 2);
              const int seg = lane & 3;
              const float4 val = *reinterpret_cast<const float4*>(stage + r * 20 + seg * 4);
              const int row_r = __shfl_sync(0xffffffffu, row, r);
              if (row_r >= 0 && FMOE_ROW_OK(p, row_r))
                *reinterpret_cast<float4*>(obase + static_cast<size_t>(row_r) * p.ld_out + ch * 16 + seg * 4) = val;
            }
          }
        }
      }
    }
    if (!ok && threadIdx.x == 128) atomicExch(p.status, kStatusGemmTimeout | 0x23);
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
