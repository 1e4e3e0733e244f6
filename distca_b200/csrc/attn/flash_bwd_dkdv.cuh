// Core attention backward, part 1 of 2: dK and dV (sm_100a, tcgen05 / TMEM / TMA).
// The reference calls flash-attn's varlen backward and then sums the K/V gradients of duplicated contexts
// with a separate kernel (distca/runtime/megatron/ops/fused_comm_attn.py:204-279, csrc/core/memcpy.cu:159-236);
// here a context is stored once per server, so there is nothing to de-duplicate.
//
// One CTA owns one 128-key tile of one document context for one KV head and walks over every
// (query head of the GQA group, query tile) that can see it. Four tensor-core products per step:
//
//   S^T  = K  Q^T        (SS)  keys on TMEM lanes, queries on columns
//   dP^T = V  dO^T       (SS)
//   dV  += P^T  dO       (TS)  P^T  = exp2(S^T*c - LSE) written over S^T as bf16
//   dK  += dS^T Q        (TS)  dS^T = P^T o (dP^T - delta) * scale written over dP^T as bf16
//   (each thread packs into the first half of its own 32 columns, so the 16 queries of K-step kk
//    sit at column 32 (kk / 2) + 8 (kk % 2) and no thread overwrites what another still reads)
//
// Both "A" operands of the accumulating products come straight from TMEM, so per step the shared
// memory only feeds K/Q and V/dO once and dO / Q once more as "B" operands; nothing is staged
// through shared memory by the threads. dK and dV stay in TMEM for the whole walk and are stored
// once: a key tile belongs to exactly one CTA and the GQA group is reduced inside it, so there
// are no atomics and the result is bit-reproducible. dQ is computed by the query-centred kernel
// in flash_bwd_dq.cuh.
//
// The tensor core never waits for a thread hand-shake it does not need: S^T(i+1) is issued right
// behind dV(i) and dP^T(i+1) right behind dK(i) (tcgen05.mma executes in issue order, so the
// overwritten P^T / dS^T have been consumed).
//
// TMEM columns: [0,128) S^T / P^T, [128,256) dP^T / dS^T, [256,384) dV, [384,512) dK.
// Warps 0-15 compute (TMEM lane quarter = warp % 4; warp group warp / 4 owns query columns
// 32 * (warp / 4) .. + 31; four warps per scheduler hide one another's TMEM-load, exponential and
// barrier latencies), warp 16 = TMA producer + per-tile LSE/delta loader, warp 17 = MMA issuer.
#pragma once
#include "../common/host_utils.h"
#include "../common/ptx.cuh"
#include "attn_common.cuh"

namespace dca {
namespace attn {

constexpr int kBwdCW = 16;                      // compute warps
constexpr int kBwdCols = 128 / (kBwdCW / 4);    // query columns per thread
constexpr int kBwdThreads = (kBwdCW + 2) * 32;
constexpr int kBT = 128;                    // tile edge (keys, queries)
constexpr int kBD = 128;                    // head dim
constexpr int kTileB = kBT * kBD * 2;       // 32 KiB
constexpr int kDkdvBars = 18;
// K, V, 2 x (Q | dO), 2 x (lse, delta), barriers, tmem slot, alignment slack
constexpr int kDkdvSmemUsed = 6 * kTileB + 2048 + kDkdvBars * 8 + 16;
constexpr int kDkdvSmem = kDkdvSmemUsed + 1024;

struct BwdParams {
  const BwdKVWork* kv_work;
  const BwdQTile* q_tiles;
  int heads_q, heads_kv;
  float scale;          // softmax scale
  float scale_log2;     // softmax scale * log2(e)
  const float* lse2;    // [heads_q, Tq] log-sum-exp in log2 units
  const float* delta;   // [heads_q, Tq] rowsum(dO o O)
  long Tq;
  __nv_bfloat16* dk;    // [Tk, ld_dk]
  __nv_bfloat16* dv;
  long ld_dk, ld_dv;
  // Optional: address of the dK row (KV head 0) of every K/V row, e.g. a copy slot in the token owner's
  // arena on another GPU; its dV row sits dv_off_bytes behind. 0 = row not stored. Replaces dk / dv when given.
  const unsigned long long* dkv_row_ptr;
  long dv_off_bytes;
  unsigned int* status;
};

__device__ __forceinline__ float ex2b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sK = smem_u32(smem);
  const uint32_t sV = sK + kTileB;
  const uint32_t sStage = sV + kTileB;        // stage s: Q at +s*64K, dO at +s*64K+32K
  float* s_stats = reinterpret_cast<float*>(smem + 6 * kTileB);  // [2][lse 128 | delta 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileB + 2048);
  const uint32_t bar_kv = smem_u32(bars);
  const uint32_t bar_qfull = bar_kv + 8;          // [2]
  const uint32_t bar_dofull = bar_qfull + 16;     // [2]
  const uint32_t bar_qdoempty = bar_dofull + 16;  // [2]
  const uint32_t bar_spare0 = bar_qdoempty + 16;
  const uint32_t bar_dpfull = bar_spare0 + 8;
  const uint32_t bar_pready = bar_dpfull + 8;
  const uint32_t bar_dsready = bar_pready + 8;
  const uint32_t bar_accfull = bar_dsready + 8;
  // [2] by step parity; two arrivals each: S^T committed by the tensor core and the step's LSE / delta
  // rows written by the loader warp, so the compute warps poll one barrier instead of two
  const uint32_t bar_sfull = bar_accfull + 8;
  const uint32_t bar_stempty = bar_sfull + 16;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kDkdvBars);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const BwdKVWork w = p.kv_work[blockIdx.x];
  const int kv_head = blockIdx.y;
  const int group = p.heads_q / p.heads_kv;
  const int n_qt = w.qt_end - w.qt_begin;
  const int n_iter = n_qt * group;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qfull + s * 8, 1);
      mbar_init(bar_dofull + s * 8, 1);
      mbar_init(bar_qdoempty + s * 8, 1);
      mbar_init(bar_sfull + s * 8, 2);
      mbar_init(bar_stempty + s * 8, kBwdCW);
    }
    (void)bar_spare0;
    mbar_init(bar_dpfull, 1);
    mbar_init(bar_pready, kBwdCW);
    mbar_init(bar_dsready, kBwdCW);
    mbar_init(bar_accfull, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == kBwdCW + 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  bool aborted = false;

  if (warp == kBwdCW) {
    // ------------------- TMA producer + per-tile statistics loader (whole warp) -------------------
    const int kcol = kv_head * kBD;
    if (lane == 0 && n_iter > 0) {
      mbar_arrive_expect_tx(bar_kv, 2 * kTileB);
      tma_load_2d(sK, &tmK, bar_kv, kcol, w.k_row0);
      tma_load_2d(sK + kBT * 128, &tmK, bar_kv, kcol + 64, w.k_row0);
      tma_load_2d(sV, &tmV, bar_kv, kcol, w.k_row0);
      tma_load_2d(sV + kBT * 128, &tmV, bar_kv, kcol + 64, w.k_row0);
    }
    for (int i = 0; i < n_iter; ++i) {
      const int s = i & 1;
      const uint32_t ph = (uint32_t)(i >> 1) & 1u;
      const int head = kv_head * group + i / n_qt;
      const BwdQTile qt = p.q_tiles[w.qt_begin + i % n_qt];
      // statistics of the query tile: lse (log2 units) and delta, +inf / 0 for rows past the task
      if (!mbar_wait_warp(bar_stempty + s * 8, ph ^ 1u, p.status)) { aborted = true; break; }
      float* st = s_stats + s * 256;
      const long idx = (long)head * p.Tq + qt.q_row0;
#pragma unroll
      for (int j = lane; j < kBT; j += 32) {
        const bool ok = j < qt.q_valid;
        st[j] = ok ? -p.lse2[idx + j] : -INFINITY;             // exp2(s*c + this)
        st[kBT + j] = ok ? -p.delta[idx + j] * p.scale : 0.f;  // dS = P * (dP*scale + this)
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sfull + s * 8);
      if (!mbar_wait_warp(bar_qdoempty + s * 8, ph ^ 1u, p.status)) { aborted = true; break; }
      if (lane == 0) {
        const int col = head * kBD;
        const uint32_t q_dst = sStage + s * 2 * kTileB, do_dst = q_dst + kTileB;
        mbar_arrive_expect_tx(bar_qfull + s * 8, kTileB);
        tma_load_2d(q_dst, &tmQ, bar_qfull + s * 8, col, qt.q_row0);
        tma_load_2d(q_dst + kBT * 128, &tmQ, bar_qfull + s * 8, col + 64, qt.q_row0);
        mbar_arrive_expect_tx(bar_dofull + s * 8, kTileB);
        tma_load_2d(do_dst, &tmdO, bar_dofull + s * 8, col, qt.q_row0);
        tma_load_2d(do_dst + kBT * 128, &tmdO, bar_dofull + s * 8, col + 64, qt.q_row0);
      }
    }
  } else if (warp == kBwdCW + 1) {
    // ------------------------------ MMA issuer ------------------------------
    // The whole warp runs this loop (warp-uniform control flow, so smem descriptors are plain
    // adds on uniform values); only the elected lane issues tcgen05.mma / tcgen05.commit.
    {
      const uint32_t leader = elect_one();
      constexpr uint32_t idesc_kk = make_idesc_bf16(kBT, kBT, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_kmn = make_idesc_bf16(kBT, kBD, 0, 1);  // dV, dK (A from TMEM, B MN-major)
      const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 384;
      const uint64_t dsc_k = make_sdesc_sw128(sK, 16, 1024), dsc_v = make_sdesc_sw128(sV, 16, 1024);
      const uint64_t dsc_st = make_sdesc_sw128(sStage, 16, 1024);            // K-major view of a stage tile
      const uint64_t dsc_stt = make_sdesc_sw128(sStage, kBT * 128, 1024);    // MN-major view
      constexpr uint64_t kTileU = (uint64_t)(kTileB >> 4);                   // one tile in descriptor units
      auto mma_kmajor = [&](uint32_t d_tmem, uint64_t a_dsc, uint64_t b_dsc) {
#pragma unroll
        for (int ks = 0; ks < kBD / 16; ++ks) {
          const uint64_t off = (uint64_t)(((ks / 4) * (kBT * 128) + (ks % 4) * 32) >> 4);
          umma_ss_p(d_tmem, a_dsc + off, b_dsc + off, idesc_kk, ks > 0 ? 1u : 0u, leader);
        }
      };
      do {
        if (n_iter == 0) break;
        if (!mbar_wait(bar_kv, 0, p.status)) { aborted = true; break; }
        if (!mbar_wait(bar_qfull, 0, p.status)) { aborted = true; break; }
        tc_fence_after();
        mma_kmajor(tS, dsc_k, dsc_st);
        umma_commit_p(bar_sfull, leader);   // step 0
        if (!mbar_wait(bar_dofull, 0, p.status)) { aborted = true; break; }
        tc_fence_after();
        mma_kmajor(tdP, dsc_v, dsc_st + kTileU);
        umma_commit_p(bar_dpfull, leader);
        for (int i = 0; i < n_iter; ++i) {
          const int s = i & 1, s1 = s ^ 1;
          const uint32_t par = (uint32_t)i & 1u;
          // stage s: Q at tile 2s, dO at tile 2s + 1
          const uint64_t q_s = dsc_stt + (uint64_t)(2 * s) * kTileU, do_s = q_s + kTileU;
          const uint64_t q_n = dsc_st + (uint64_t)(2 * s1) * kTileU, do_n = q_n + kTileU;
          // dV += P^T dO : A = P^T from TMEM, B = dO viewed [d, q] (MN-major)
          if (!mbar_wait(bar_pready, par, p.status)) { aborted = true; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kBT / 16; ++kk)
            umma_ts_p(tdV, tS + (kk / 2) * 32 + (kk % 2) * 8, do_s + (uint64_t)((kk * 2048) >> 4), idesc_kmn,
                      (i > 0 || kk > 0) ? 1u : 0u, leader);
          if (i + 1 < n_iter) {
            if (!mbar_wait(bar_qfull + s1 * 8, (uint32_t)((i + 1) >> 1) & 1u, p.status)) { aborted = true; break; }
            tc_fence_after();
            mma_kmajor(tS, dsc_k, q_n);
            umma_commit_p(bar_sfull + s1 * 8, leader);
          }
          // dK += dS^T Q : A = dS^T from TMEM, B = Q viewed [d, q] (MN-major)
          if (!mbar_wait(bar_dsready, par, p.status)) { aborted = true; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kBT / 16; ++kk)
            umma_ts_p(tdK, tdP + (kk / 2) * 32 + (kk % 2) * 8, q_s + (uint64_t)((kk * 2048) >> 4), idesc_kmn,
                      (i > 0 || kk > 0) ? 1u : 0u, leader);
          umma_commit_p(bar_qdoempty + s * 8, leader);
          if (i + 1 < n_iter) {
            if (!mbar_wait(bar_dofull + s1 * 8, (uint32_t)((i + 1) >> 1) & 1u, p.status)) { aborted = true; break; }
            tc_fence_after();
            mma_kmajor(tdP, dsc_v, do_n);
            umma_commit_p(bar_dpfull, leader);
          }
        }
        if (!aborted) umma_commit_p(bar_accfull, leader);
      } while (false);
      __syncwarp();
    }
  } else {
    // ------------------------------ compute warps ------------------------------
    const int cw = warp >> 2;                    // query columns cw * kBwdCols .. + kBwdCols - 1
    const int qd = warp & 3;
    const int r = qd * 32 + lane;                // TMEM lane = key row of the tile
    const uint32_t lane_base = (uint32_t)(qd * 32) << 16;
    const uint32_t tS = tmem_base + lane_base;
    const uint32_t tdP = tS + 128, tdV = tS + 256, tdK = tS + 384;
    const int c0 = cw * kBwdCols;
    static_assert(kBwdCols == 32, "one 32-column TMEM load per thread and step");
    for (int i = 0; i < n_iter; ++i) {
      const uint32_t par = (uint32_t)i & 1u;
      const BwdQTile qt = p.q_tiles[w.qt_begin + i % n_qt];
      const float* st = s_stats + (i & 1) * 256;
      float pf[kBwdCols];
      // ---- P^T = exp2(S^T * c - lse2), masked ----
      if (!mbar_wait_warp(bar_sfull + (i & 1) * 8, (uint32_t)(i >> 1) & 1u, p.status)) { aborted = true; break; }
      tc_fence_after();
      {
        uint32_t sv[32];
        tmem_ld32(tS + c0, sv);
        tmem_ld_wait();
        // st[0..127] holds -lse2 per query column (-inf past the task: exp2 gives an exact 0)
        const float4* nl4 = reinterpret_cast<const float4*>(st + c0);
        if (qt.diag >= kBT - 1) {
          // every key of the tile is visible to every query of the tile: no compares at all
#pragma unroll
          for (int c4 = 0; c4 < kBwdCols / 4; ++c4) {
            const float4 nl = nl4[c4];
            const int c = c4 * 4;
            pf[c + 0] = ex2_col(fmaf(__uint_as_float(sv[c + 0]), p.scale_log2, nl.x), c + 0);
            pf[c + 1] = ex2_col(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, nl.y), c + 1);
            pf[c + 2] = ex2_col(fmaf(__uint_as_float(sv[c + 2]), p.scale_log2, nl.z), c + 2);
            pf[c + 3] = ex2_col(fmaf(__uint_as_float(sv[c + 3]), p.scale_log2, nl.w), c + 3);
          }
        } else {
#pragma unroll
          for (int c = 0; c < kBwdCols; ++c) {
            float v = ex2_col(fmaf(__uint_as_float(sv[c]), p.scale_log2, st[c0 + c]), c);
            if (r > c0 + c + qt.diag) v = 0.f;   // select: a masked score may be anything
            pf[c] = v;
          }
        }
        uint32_t pk[kBwdCols / 2];
#pragma unroll
        for (int c = 0; c < kBwdCols / 2; ++c) pk[c] = pack_bf16x2(pf[2 * c], pf[2 * c + 1]);
        // packed P^T goes into the first half of the columns this thread read its S^T from: no
        // other thread touches them, so no barrier is needed in front of the store
        tmem_st16(tS + c0, pk);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pready);
      // ---- dS^T = P^T o (dP^T - delta) * scale, written over dP^T as bf16 ----
      if (!mbar_wait_warp(bar_dpfull, par, p.status)) { aborted = true; break; }
      tc_fence_after();
      {
        uint32_t dv[32];
        tmem_ld32(tdP + c0, dv);
        tmem_ld_wait();
        uint32_t pk[kBwdCols / 2];
        // st[128..255] holds -delta * scale per query column: dS = P * (dP * scale - delta * scale)
        const float4* nd4 = reinterpret_cast<const float4*>(st + kBT + c0);
#pragma unroll
        for (int c4 = 0; c4 < kBwdCols / 4; ++c4) {
          const float4 nd = nd4[c4];
          const int c = c4 * 4;
          const float t0 = pf[c + 0] * fmaf(__uint_as_float(dv[c + 0]), p.scale, nd.x);
          const float t1 = pf[c + 1] * fmaf(__uint_as_float(dv[c + 1]), p.scale, nd.y);
          const float t2 = pf[c + 2] * fmaf(__uint_as_float(dv[c + 2]), p.scale, nd.z);
          const float t3 = pf[c + 3] * fmaf(__uint_as_float(dv[c + 3]), p.scale, nd.w);
          pk[c / 2] = pack_bf16x2(t0, t1);
          pk[c / 2 + 1] = pack_bf16x2(t2, t3);
        }
        tmem_st16(tdP + c0, pk);   // own columns again
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bar_dsready);
        mbar_arrive(bar_stempty + (i & 1) * 8);
      }
    }
    // ---- epilogue: dK, dV (this warp group stores head-dim columns c0 .. c0 + 31) ----
    if (!aborted && n_iter > 0) {
      if (mbar_wait_warp(bar_accfull, 0, p.status)) {
        tc_fence_after();
        bool row_ok = r < w.k_valid;
        __nv_bfloat16 *dk_row, *dv_row;
        if (p.dkv_row_ptr != nullptr) {
          const unsigned long long rowp = row_ok ? p.dkv_row_ptr[(long)w.k_row0 + r] : 0ull;
          row_ok = rowp != 0ull;
          dk_row = reinterpret_cast<__nv_bfloat16*>(rowp) + (long)kv_head * kBD + c0;
          dv_row = reinterpret_cast<__nv_bfloat16*>(rowp + (unsigned long long)p.dv_off_bytes) + (long)kv_head * kBD + c0;
        } else {
          dk_row = p.dk + ((long)w.k_row0 + r) * p.ld_dk + (long)kv_head * kBD + c0;
          dv_row = p.dv + ((long)w.k_row0 + r) * p.ld_dv + (long)kv_head * kBD + c0;
        }
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          uint32_t a[32];
          tmem_ld32((which == 0 ? tdK : tdV) + c0, a);
          tmem_ld_wait();
          if (row_ok) {
            __nv_bfloat16* dst = which == 0 ? dk_row : dv_row;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 u;
              const int b = v * 8;
              u.x = pack_bf16x2(__uint_as_float(a[b + 0]), __uint_as_float(a[b + 1]));
              u.y = pack_bf16x2(__uint_as_float(a[b + 2]), __uint_as_float(a[b + 3]));
              u.z = pack_bf16x2(__uint_as_float(a[b + 4]), __uint_as_float(a[b + 5]));
              u.w = pack_bf16x2(__uint_as_float(a[b + 6]), __uint_as_float(a[b + 7]));
              *reinterpret_cast<uint4*>(dst + b) = u;
            }
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
  if (warp == kBwdCW + 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace attn
}  // namespace dca
