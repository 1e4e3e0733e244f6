// Core attention backward, part 2 of 2: dQ (sm_100a, tcgen05 / TMEM / TMA).
// The reference calls flash-attn's varlen backward for this (distca/runtime/megatron/ops/fused_comm_attn.py:204-279).
//
// One CTA owns one 128-row query tile of one core-attention task for one query head and streams
// the key tiles it can see (the same work list as the forward pass). Three products per key tile:
//
//   S   = Q  K^T         (SS)  queries on TMEM lanes, keys on columns; double-buffered
//   dP  = dO V^T         (SS)
//   dQ += dS K           (TS)  dS = exp2(S*c - LSE) o (dP - delta) * scale as bf16,
//                              K viewed [d, keys] (MN-major) from the tile already in shared memory
//
// dQ accumulates in TMEM over the whole walk and is stored once as bf16: no atomics, no fp32
// accumulation buffer, bit-reproducible. LSE and delta belong to the thread's own row, so they
// live in two registers.
//
// dS(j) is written into the S buffer that held S(j), in the columns the same thread read its scores
// from (no cross-thread hazard, so no barrier in front of the store); the dP columns are free as soon
// as the tile's threads have loaded dP(j) and dP(j+1) is issued at that moment; S(j+2) follows dQ(j)
// into the same buffer (tcgen05.mma executes in issue order).
//
// The compute warps form two groups that take alternate key tiles (group g: tiles g, g+2, ...; it
// always uses S buffer g). While one group waits on barriers, loads TMEM and packs dS, the other is
// in its exponentials, so the MUFU pipe - the scarce thread-side resource - stays busy, and a
// barrier poll queued behind another warp's MUFU burst delays only its own group.
// K is triple-buffered because S(j+2) is issued before dQ(j+1) has read K(j+1).
//
// TMEM columns: [0,128) S / dS buffer 0, [128,256) S / dS buffer 1, [256,384) dP, [384,512) dQ.
// Warps 0-15 compute: TMEM lane quarter = warp % 4, group = warp / 8, key columns
// 64 * ((warp / 4) % 2) .. + 63; warp 16 = TMA producer, warp 17 = MMA issuer.
#pragma once
#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "attn_common.cuh"

namespace dca {
namespace attn {

constexpr int kDqCW = 16;                       // compute warps
constexpr int kDqCols = 64;                     // key columns per thread (two groups x two halves)
constexpr int kDqGW = kDqCW / 2;                // warps per group
constexpr int kDqThreads = (kDqCW + 2) * 32;
constexpr int kDqKStages = 3;
constexpr int kDqVStages = 2;
constexpr int kDqBars = 1 + 2 * kDqKStages + 2 * kDqVStages + 4 * 2 + 1;
// Q, dO, 3 x K, 2 x V, barriers, tmem slot, alignment slack
constexpr int kDqSmemUsed = (2 + kDqKStages + kDqVStages) * 32768 + kDqBars * 8 + 16;
constexpr int kDqSmem = kDqSmemUsed + 1024;


struct DqParams {
  const AttnWork* work;
  int heads_q, heads_kv;
  float scale, scale_log2;
  const float* lse2;    // [heads_q, Tq]
  const float* delta;   // [heads_q, Tq]
  long Tq;
  __nv_bfloat16* dq;    // [Tq, ld_dq]
  long ld_dq;
  // Optional: address of the dQ row (head 0) of every Q row, e.g. in the token owner's arena on another GPU
  // (plain peer stores over NVLink); 0 = row not stored. Replaces dq / ld_dq when given.
  const unsigned long long* dq_row_ptr;
  unsigned int* status;
};

__global__ void __launch_bounds__(kDqThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const DqParams p) {
  constexpr int T = 128, D = 128, TILE = 32768;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sdO = sQ + TILE;
  const uint32_t sK = sdO + TILE;                       // kDqKStages tiles
  const uint32_t sV = sK + kDqKStages * TILE;           // kDqVStages tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + kDqKStages + kDqVStages) * TILE);
  const uint32_t bar_q = smem_u32(bars);
  const uint32_t bar_kfull = bar_q + 8;                           // [3]
  const uint32_t bar_kempty = bar_kfull + kDqKStages * 8;         // [3]
  const uint32_t bar_vfull = bar_kempty + kDqKStages * 8;         // [2]
  const uint32_t bar_vempty = bar_vfull + kDqVStages * 8;         // [2]
  const uint32_t bar_sfull = bar_vempty + kDqVStages * 8;         // [2]
  const uint32_t bar_dpfull = bar_sfull + 16;                     // [2] by tile parity
  const uint32_t bar_ldp = bar_dpfull + 16;                       // [2] the tile's group has loaded dP
  const uint32_t bar_dsready = bar_ldp + 16;                      // [2]
  const uint32_t bar_dqfull = bar_dsready + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kDqBars);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const AttnWork w = p.work[blockIdx.x];
  const int head = blockIdx.y;
  const int kv_head = head / (p.heads_q / p.heads_kv);
  const int n_kv = (w.kv_limit_base + w.q_valid + T - 1) / T;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kDqKStages; ++s) {
      mbar_init(bar_kfull + s * 8, 1);
      mbar_init(bar_kempty + s * 8, 1);
    }
    for (int s = 0; s < kDqVStages; ++s) {
      mbar_init(bar_vfull + s * 8, 1);
      mbar_init(bar_vempty + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_sfull + b * 8, 1);
      mbar_init(bar_dpfull + b * 8, 1);
      mbar_init(bar_ldp + b * 8, kDqGW);
      mbar_init(bar_dsready + b * 8, kDqGW);
    }
    mbar_init(bar_dqfull, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == kDqCW + 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  bool aborted = false;

  if (warp == kDqCW) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      const int qcol = head * D, kcol = kv_head * D;
      mbar_arrive_expect_tx(bar_q, 2 * TILE);
      tma_load_2d(sQ, &tmQ, bar_q, qcol, w.q_row0);
      tma_load_2d(sQ + T * 128, &tmQ, bar_q, qcol + 64, w.q_row0);
      tma_load_2d(sdO, &tmdO, bar_q, qcol, w.q_row0);
      tma_load_2d(sdO + T * 128, &tmdO, bar_q, qcol + 64, w.q_row0);
      for (int j = 0; j < n_kv; ++j) {
        const int ks = j % kDqKStages, vs = j % kDqVStages;
        const int krow = w.k_row0 + j * T;
        if (!mbar_wait(bar_kempty + ks * 8, ((uint32_t)(j / kDqKStages) & 1u) ^ 1u, p.status)) { aborted = true; break; }
        mbar_arrive_expect_tx(bar_kfull + ks * 8, TILE);
        tma_load_2d(sK + ks * TILE, &tmK, bar_kfull + ks * 8, kcol, krow);
        tma_load_2d(sK + ks * TILE + T * 128, &tmK, bar_kfull + ks * 8, kcol + 64, krow);
        if (!mbar_wait(bar_vempty + vs * 8, ((uint32_t)(j / kDqVStages) & 1u) ^ 1u, p.status)) { aborted = true; break; }
        mbar_arrive_expect_tx(bar_vfull + vs * 8, TILE);
        tma_load_2d(sV + vs * TILE, &tmV, bar_vfull + vs * 8, kcol, krow);
        tma_load_2d(sV + vs * TILE + T * 128, &tmV, bar_vfull + vs * 8, kcol + 64, krow);
      }
    }
  } else if (warp == kDqCW + 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs this loop (warp-uniform control flow, so smem descriptors are plain
    // adds on uniform values); only the elected lane issues tcgen05.mma / tcgen05.commit.
    {
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc_kk = make_idesc_bf16(T, T, 0, 0);   // S, dP
      constexpr uint32_t idesc_dq = make_idesc_bf16(T, D, 0, 1);   // dQ: A from TMEM, B = K MN-major
      const uint32_t tdP = tmem_base + 256, tdQ = tmem_base + 384;
      const uint64_t dsc_q = make_sdesc_sw128(sQ, 16, 1024), dsc_do = make_sdesc_sw128(sdO, 16, 1024);
      const uint64_t dsc_k0 = make_sdesc_sw128(sK, 16, 1024);            // K-major view (S)
      const uint64_t dsc_k0t = make_sdesc_sw128(sK, T * 128, 1024);      // MN-major view (dQ)
      const uint64_t dsc_v0 = make_sdesc_sw128(sV, 16, 1024);
      // D = A B^T over the head dim; descriptor offsets are in 16-byte units
      auto mma_kmajor = [&](uint32_t d_tmem, uint64_t a_dsc, uint64_t b_dsc) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint64_t off = (uint64_t)(((ks / 4) * (T * 128) + (ks % 4) * 32) >> 4);
          umma_ss_p(d_tmem, a_dsc + off, b_dsc + off, idesc_kk, ks > 0 ? 1u : 0u, leader);
        }
      };
      // S(j) into buffer j & 1. Its previous content dS(j-2) was consumed by dQ(j-2), issued earlier.
      auto issue_s = [&](int j) -> bool {
        const int ks = j % kDqKStages;
        if (!mbar_wait(bar_kfull + ks * 8, (uint32_t)(j / kDqKStages) & 1u, p.status)) return false;
        tc_fence_after();
        mma_kmajor(tmem_base + (j & 1) * T, dsc_q, dsc_k0 + (uint64_t)((ks * TILE) >> 4));
        umma_commit_p(bar_sfull + (j & 1) * 8, leader);
        return true;
      };
      auto issue_dp = [&](int j) -> bool {
        const int vs = j % kDqVStages;
        if (!mbar_wait(bar_vfull + vs * 8, (uint32_t)(j / kDqVStages) & 1u, p.status)) return false;
        tc_fence_after();
        mma_kmajor(tdP, dsc_do, dsc_v0 + (uint64_t)((vs * TILE) >> 4));
        umma_commit_p(bar_dpfull + (j & 1) * 8, leader);
        umma_commit_p(bar_vempty + vs * 8, leader);
        return true;
      };
      do {
        if (!mbar_wait(bar_q, 0, p.status)) { aborted = true; break; }
        if (!issue_s(0)) { aborted = true; break; }
        if (!issue_dp(0)) { aborted = true; break; }
        if (n_kv > 1 && !issue_s(1)) { aborted = true; break; }
        for (int j = 0; j < n_kv; ++j) {
          const uint32_t par = (uint32_t)(j >> 1) & 1u;
          const int g = j & 1;
          // dP(j+1) as soon as the threads of tile j have read dP(j)
          if (j + 1 < n_kv) {
            if (!mbar_wait(bar_ldp + g * 8, par, p.status)) { aborted = true; break; }
            if (!issue_dp(j + 1)) { aborted = true; break; }
          }
          // dQ += dS(j) K(j); dS of keys 16kk.. sits where their scores sat: column 64 (kk/4) + 8 (kk%4)
          if (!mbar_wait(bar_dsready + g * 8, par, p.status)) { aborted = true; break; }
          tc_fence_after();
          const uint64_t kb = dsc_k0t + (uint64_t)(((j % kDqKStages) * TILE) >> 4);
          const uint32_t tdS = tmem_base + g * T;
#pragma unroll
          for (int kk = 0; kk < T / 16; ++kk)
            umma_ts_p(tdQ, tdS + (kk / 4) * 64 + (kk % 4) * 8, kb + (uint64_t)((kk * 2048) >> 4), idesc_dq,
                      (j > 0 || kk > 0) ? 1u : 0u, leader);
          umma_commit_p(bar_kempty + (j % kDqKStages) * 8, leader);
          if (j + 2 < n_kv && !issue_s(j + 2)) { aborted = true; break; }
        }
        if (!aborted) umma_commit_p(bar_dqfull, leader);
      } while (false);
      __syncwarp();
    }
  } else {
    // ------------------------------ compute warps ------------------------------
    const int g = warp / kDqGW;                  // tile parity this warp works on = its S buffer
    const int hcol = (warp >> 2) & 1;            // key-column half
    const int qd = warp & 3;
    const int r = qd * 32 + lane;                // TMEM lane = query row of the tile
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + g * T;    // S buffer of this group's tiles
    const uint32_t tdP = tmem_base + lane_base + 256, tdQ = tmem_base + lane_base + 384;
    const int c0 = hcol * kDqCols;
    const bool row_ok = r < w.q_valid;
    const long sidx = (long)head * p.Tq + w.q_row0 + r;
    const float nlse = row_ok ? -p.lse2[sidx] : -INFINITY;         // P = exp2(S*c + nlse)
    const float ndelta = row_ok ? -p.delta[sidx] * p.scale : 0.f;   // dS = P * (dP*scale + ndelta)
    const int limit = w.kv_limit_base + r;       // last key this row may see
    for (int j = g; j < n_kv; j += 2) {
      const uint32_t par = (uint32_t)(j >> 1) & 1u;
      float pf[kDqCols];
      // ---- P = exp2(S * c - lse2), masked ----
      if (!mbar_wait_warp(bar_sfull + g * 8, par, p.status)) { aborted = true; break; }
      tc_fence_after();
      const bool full_tile = j * T + T - 1 <= w.kv_limit_base;   // every key visible to every row
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t sv[32];
        tmem_ld32(tS + c0 + hh * 32, sv);
        tmem_ld_wait();

        const int key0 = j * T + c0 + hh * 32;
        if (full_tile) {
#pragma unroll
          for (int c = 0; c < 32; ++c)
            pf[hh * 32 + c] = ex2_col(fmaf(__uint_as_float(sv[c]), p.scale_log2, nlse), c);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float v = ex2_col(fmaf(__uint_as_float(sv[c]), p.scale_log2, nlse), c);
            if (key0 + c > limit) v = 0.f;   // select: masked keys may hold anything
            pf[hh * 32 + c] = v;
          }
        }
      }
      // ---- dS = P o (dP - delta) * scale as bf16, into the columns this thread read S from ----
      if (!mbar_wait_warp(bar_dpfull + g * 8, par, p.status)) { aborted = true; break; }
      tc_fence_after();
      // eight-column steps keep the live registers under the 96 a 576-thread CTA may use
#pragma unroll
      for (int q8 = 0; q8 < 8; ++q8) {
        uint32_t dv[8];
        tmem_ld8(tdP + c0 + q8 * 8, dv);
        tmem_ld_wait();
        if (q8 == 7) {
          // the dP columns may now be overwritten by dP(j+1)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_ldp + g * 8);
        }
        uint32_t pk[4];
#pragma unroll
        for (int c = 0; c < 8; c += 2) {
          const float t0 = pf[q8 * 8 + c] * fmaf(__uint_as_float(dv[c]), p.scale, ndelta);
          const float t1 = pf[q8 * 8 + c + 1] * fmaf(__uint_as_float(dv[c + 1]), p.scale, ndelta);
          pk[c / 2] = pack_bf16x2(t0, t1);
        }
        tmem_st4(tS + c0 + q8 * 4, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_dsready + g * 8);
    }
    const int cw = warp >> 2;
    const int e0 = cw * 32;                      // epilogue: head-dim columns of this warp
    // ---- epilogue: dQ (this warp group stores head-dim columns c0 .. c0 + 31) ----
    if (!aborted) {
      if (mbar_wait_warp(bar_dqfull, 0, p.status)) {
        tc_fence_after();
        uint32_t a[32];
        tmem_ld32(tdQ + e0, a);
        tmem_ld_wait();
        unsigned long long rowp = 1ull;
        if (row_ok && p.dq_row_ptr != nullptr) rowp = p.dq_row_ptr[(long)w.q_row0 + r];
        if (row_ok && rowp != 0ull) {
          __nv_bfloat16* dst = p.dq_row_ptr != nullptr
                                   ? reinterpret_cast<__nv_bfloat16*>(rowp) + (long)head * D + e0
                                   : p.dq + ((long)w.q_row0 + r) * p.ld_dq + (long)head * D + e0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 u;
            const int bb = v * 8;
            u.x = pack_bf16x2(__uint_as_float(a[bb + 0]), __uint_as_float(a[bb + 1]));
            u.y = pack_bf16x2(__uint_as_float(a[bb + 2]), __uint_as_float(a[bb + 3]));
            u.z = pack_bf16x2(__uint_as_float(a[bb + 4]), __uint_as_float(a[bb + 5]));
            u.w = pack_bf16x2(__uint_as_float(a[bb + 6]), __uint_as_float(a[bb + 7]));
            *reinterpret_cast<uint4*>(dst + bb) = u;
          }
        }
      } else {
        aborted = true;
      }
    }
  }

  if (aborted) {
    for (int i = 0; i < 256; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kDqCW + 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace attn
}  // namespace dca
