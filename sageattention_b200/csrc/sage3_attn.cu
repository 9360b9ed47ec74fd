// Block-scaled FP4 attention for sm_100a: TMA-staged E2M1 tiles, tcgen05 NVFP4 MMAs with the S and O
// accumulators in tensor memory, exp2 online softmax, P re-quantized to NVFP4 before the PV MMA.
//
// One CTA per PAIR of 128-row query tiles of one head; every K / V^T stage in shared memory serves both
// tiles.  Six warpgroups (setmaxnreg moves registers to the softmax warpgroups):
//   warp 0       TMA producer (one lane): both Q tiles once, then K (+ one delta_s row per tile) / V^T /
//                scale atoms per KV block
//   warp 1       Q K^T MMA issuer (one lane) and owner of the tensor-memory allocation
//   warp 2       P V MMA issuer (one lane); warp 3 idle
//   warps 4-11   softmax of query tile 0, warps 12-19 softmax of query tile 1.  A row is shared by two threads
//                (same lane quarter, different warpgroups): thread h owns keys [64 h, 64 h + 64) of every KV
//                block and, in the epilogue, columns [D/2 h, D/2 (h + 1)) of the O row.
//   warps 20-23  O rescale ("correction"), one warp per tensor-memory lane quarter: when a row of the quarter moved
//                its maximum, the warp multiplies the 32 O rows of its quarter by their factors before the block's
//                P V MMA is issued.  The softmax warps hand the factors over through shared memory and never touch
//                O inside the loop, so neither the wait for the previous P V nor the tensor-memory round trip sits
//                in their instruction stream.
// Per KV block a softmax thread pulls its 64 scores out of tensor memory into registers (the S buffer goes to
// the other tile as soon as all eight warps have done so) and runs the exp2 pass at once, microblock by microblock,
// the maxima of the next microblock found under the exponentials of the current one: with
// E = P~ / sf = 6 * 2^((S - bm) s), the exp2 values and FP4 codes of a microblock depend on the maximum bm of that
// microblock only.  The running row maximum enters just the E4M3 scales, the row
// sum and the O rescale factor; the two threads of a row exchange their half maxima through shared memory
// (published before the pass, read after it), so the exchange costs no wait.  Then the thread stores its half
// of the P row (codes + scales) and at the end writes its half of O / l.
// Tensor memory (512 columns) holds one 128-column S buffer, the two O accumulators and the scale factors; the
// S buffer alternates between the tiles, which keeps the two tiles half a block apart: one pair of warps per
// scheduler is in its exp2 pass while the other pair loads, reduces and stores.
//
// Arithmetic follows (paths inside the reference project, sageattention3_blackwell/sageattn3/blackwell/...):
//   mainloop_tma_ws.h:509, 532-551, 865     KV blocks are walked from the last to the first
//   mainloop_tma_ws.h:691-704, 718          S starts from the delta_s row of the query tile (here: a rank-1
//                                           16-bit MMA, ones (x) delta_s, issued before the FP4 MMAs)
//   mainloop_tma_ws.h:732-748               masks (applied here on the real key index)
//   softmax_fused.h:39-137                  running max per 128 keys, P~ = 2^(S s - m s) * 2688, row sum of the
//                                           unquantized P~, microblock scale max(P~)/6 (E4M3 in the MMA)
//   softmax_fused.h:139-170                 O = O alpha + P^ V^;  out = O / l  (0 when l == 0)
// Every wait is bounded (see mbar_wait); a wait that gives up records a code in the status word and the
// CTA winds down without touching tensor memory it does not own.
#include <cuda.h>

#include <type_traits>

#include "sage3_common.cuh"
#include "sage3_kernels.h"

namespace sage3 {

// Development instrumentation (compiled only with -DSAGE3_DEV_TRACE; the product library has none of it):
// per-phase cycle sums of every softmax warp of the first CTA, a time line of a few KV blocks, and a dump of
// the first block's scores, statistics and accumulators of the first query tile.
#ifdef SAGE3_DEV_TRACE
#define PT_DECL long long pt_t = clock64(); long long pt_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define PT(i) { const long long pt_now = clock64(); pt_acc[i] += pt_now - pt_t; pt_t = pt_now; }
#define PT_DUMP(slot) if (p.debug != nullptr && blockIdx.x == 0 && lane == 0) { for (int i_ = 0; i_ < 8; ++i_) p.debug[40000 + (slot) * 8 + i_] = (float)pt_acc[i_]; }
// time line: event `ev` (0..15) of actor `who` (0..23) at loop index `it`, for kTrIters iterations from kTrFirst on
constexpr int kTrFirst = 40, kTrIters = 4;
#define TR(who, it, ev) if (p.debug != nullptr && blockIdx.x == 0 && lane == 0 && (it) >= kTrFirst && (it) < kTrFirst + kTrIters) \
    { p.debug[42000 + ((who) * kTrIters + ((it) - kTrFirst)) * 16 + (ev)] = __uint_as_float((uint32_t)clock64()); }
#define DEV_DUMP(...) __VA_ARGS__
#else
#define PT_DECL
#define PT(i)
#define PT_DUMP(slot)
#define TR(who, it, ev)
#define DEV_DUMP(...)
#endif

constexpr float kLog2Of6 = 2.584962500721156f;
constexpr float kPScaleLog2 = -11.392317422778762f;   // log2(1 / (448 * 6)), softmax_fused.h:33

struct AttnParams {
    int Hq, Hkv, Nq, Nk, nqt, nkb, nqm;   // nqt = query tiles per head, nkb = KV blocks per head
    float sm_scale_log2;
    const float* sm_scale_per_head;
    const uint8_t *q_sf, *k_sf, *v_sf;
    const uint16_t* delta;              // 16-bit elements [B*Hq][nqm][nkb*128]
    void* out[kMaxParts];               // output buffers; out_rows == 0: one buffer
    int out_rows;                       // query rows per output part (rows of one (batch, head) go to part row / out_rows)
    int64_t os0, os1, os2;
    float* lse;                         // optional fp32 [B*Hq][Nq]
    const float* qkm;                   // fp32 [B*Hq][nqt*128]: q . km per query row
    float sm_scale;
    int* status;
    const int* prepass_status;
    // accumulator state carried between calls that walk consecutive key ranges of one attention (nullptr: none)
    const float *carry_o_in, *carry_m_in, *carry_l_in;   // fp32 [B*Hq][Nq][D] unnormalized O; [B*Hq][Nq] running max; [B*Hq][Nq][2] partial row sums
    float *carry_o_out, *carry_m_out, *carry_l_out;
    int causal_shift;                   // key j is visible to query i iff j <= i + causal_shift
    const int *cu_q, *cu_k;             // packed variable-length sequences (VARLEN kernels): entry b owns rows cu[b] .. cu[b + 1]
#ifdef SAGE3_DEV_TRACE
    float* debug;                       // development dump of CTA 0 (nullptr in normal use)
#endif
};

template <int D>
struct Cfg {
    static constexpr int kStages = 6;                         // K and V^T stages, each shared by the two query tiles
    static constexpr int kThreads = 768;                      // 6 warpgroups, see the kernel
    static constexpr int kQBytes = 128 * D / 2;               // per query tile
    static constexpr int kSfQkBytes = (D / 64) * 512;
    static constexpr int kKBytes = 128 * D / 2;
    static constexpr int kVBytes = D * 64;
    static constexpr int kSfVBytes = 1024;
    static constexpr int kDeltaBytes = 256;
    static constexpr int kPBytes = 8192;
    // shared-memory map (bytes from a 1024-aligned base)
    static constexpr int oQ = 0;                              // [tile] 8192
    static constexpr int oK = oQ + 2 * 8192;
    static constexpr int oV = oK + kStages * 8192;
    static constexpr int oP = oV + kStages * 8192;            // [tile][buffer] 8192
    static constexpr int oSfQ = oP + 4 * kPBytes;             // [tile] 1024
    static constexpr int oSfK = oSfQ + 2 * 1024;
    static constexpr int oSfV = oSfK + kStages * 1024;
    static constexpr int oSfP = oSfV + kStages * 1024;        // [tile][buffer] 1024
    static constexpr int kDeltaPitch = 512;                   // 256 B of delta_s + 256 B that stay zero
    static constexpr int oDelta = oSfP + 4 * 1024;            // [stage][tile] kDeltaPitch
    static constexpr int oOnes = oDelta + kStages * 2 * kDeltaPitch;   // 128 x 16 tile: column 0 = 1.0, rest 0
    static constexpr int oXch = oOnes + 4096;                 // float [2 parities][tile][half][128]: microblock-half maxima; [tile][half][128] row sums
    static constexpr int oBar = oXch + (8 + 4) * 128 * 4;
    static constexpr int kNumBars = 1 + 4 * kStages + 2 + 1 + 4 + 4 + 8 + 16 + 4;
    static constexpr int oMisc = oBar + kNumBars * 8;
    static constexpr int oAlpha = oMisc + 64;                 // rescale factors, float [2 block parities][2 tiles][128 rows]
    static constexpr int kSmemBytes = oAlpha + 2048 + 1024;      // + slack for the manual 1024-byte alignment
    // tensor-memory columns: one S buffer, one O accumulator per tile, scale factors
    static constexpr uint32_t cS = 0, cO = 128, cSfQ = 384, cSfK = 400, cSfV = 408, cSfP = 416;
    static constexpr uint64_t kSwzQK = (D == 128) ? kSwz64 : kSwz32;
    static constexpr uint32_t kSboQK = (D == 128) ? 512 : 256;
};

template <typename OutT> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Wait executed by a whole converged warp; the verdict is made warp-uniform so that no lane leaves a loop alone.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
    return __all_sync(0xffffffffu, ok);
}

template <int D, bool CAUSAL, typename OutT, bool VARLEN>
__global__ void __launch_bounds__(Cfg<D>::kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p) {
    using C = Cfg<D>;
    constexpr int S = C::kStages;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t sbase = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* sgen = smem_dyn + (sbase - smem_u32(smem_dyn));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // barriers
    auto bar = [&](int i) { return sbase + C::oBar + 8u * i; };
    const int bQ = 0, bKF = 1, bKE = bKF + S, bVF = bKE + S, bVE = bVF + S, bSF = bVE + S, bSE = bSF + 2,
              bPF = bSE + 1, bPV = bPF + 4, bXC = bPV + 4, bAL = bXC + 8, bOS = bAL + 16;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + C::oMisc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + C::oMisc + 8);

    // CTA -> (batch*head, pair of query tiles); heavier causal pairs are scheduled first
    const int npair = (p.nqt + 1) >> 1;
    const int bhq = blockIdx.x / npair;
    int pr = blockIdx.x % npair;
    if (CAUSAL) pr = npair - 1 - pr;
    const int mt0 = 2 * pr;
    const int b = bhq / p.Hq, hq = bhq % p.Hq;
    const int bhkv = b * p.Hkv + hq / (p.Hq / p.Hkv);
    // Lengths of this batch entry.  p.Nq, p.Nk, p.nqt, p.nkb stay the strides of the workspace layouts; with packed
    // variable-length sequences they are the maxima and the entry's own lengths come from the cu arrays.
    int Nq = p.Nq, Nk = p.Nk, nqt = p.nqt, nkb = p.nkb, shift = p.causal_shift;
    int64_t out_base = b * p.os0;
    if constexpr (VARLEN) {
        const int q0 = p.cu_q[b], k0 = p.cu_k[b];
        Nq = min(max(p.cu_q[b + 1] - q0, 0), p.Nq);
        Nk = min(max(p.cu_k[b + 1] - k0, 0), p.Nk);
        nqt = (Nq + kBlock - 1) / kBlock;
        nkb = (Nk + kBlock - 1) / kBlock;
        shift = Nk - Nq;
        out_base = (int64_t)q0 * p.os2;
    }
    const int nv = (mt0 + 1 < nqt) ? 2 : (VARLEN && mt0 >= nqt ? 0 : 1);   // query tiles this CTA really has
    // an earlier CTA of this launch gave up, or the pre-pass did (the workspace is then incomplete)
    const bool dead_launch = (*reinterpret_cast<volatile int*>(p.status) != 0) || (*reinterpret_cast<const volatile int*>(p.prepass_status) != 0);
    // KV blocks of tile t: [0, nbt[t]); the CTA walks block n = nbmax - 1 ... 0 and tile t joins at step skip[t]
    int nbt[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        int nb = nkb;
        if (CAUSAL) {
            const int max_key = min(Nk - 1, (mt0 + t) * kBlock + kBlock - 1 + shift);
            nb = max_key < 0 ? 0 : max_key / kBlock + 1;
        }
        nbt[t] = (dead_launch || t >= nv) ? 0 : nb;
    }
    const int nbmax = max(nbt[0], nbt[1]);
    const int skip[2] = {nbmax - nbt[0], nbmax - nbt[1]};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar(bQ), 1);
        for (int i = 0; i < S; ++i) {
            mbar_init(bar(bKF + i), 1);
            mbar_init(bar(bKE + i), 1);    // every Q K^T that reads K stage i is complete
            mbar_init(bar(bVF + i), 1);
            mbar_init(bar(bVE + i), 1);    // every P V that reads V stage i is complete
        }
        mbar_init(bar(bSF), 1);            // S holds the scores of tile 0's next block
        mbar_init(bar(bSF + 1), 1);        // ... of tile 1's next block
        mbar_init(bar(bSE), 8);            // the eight warps of the tile that owns S have it in registers
        for (int i = 0; i < 4; ++i) {
            mbar_init(bar(bPF + i), 8);    // [tile][buffer]: P (+ scales) written and O rescaled
            mbar_init(bar(bPV + i), 1);    // [tile][buffer]: the P V MMA that read it is complete
        }
        for (int i = 0; i < 8; ++i) mbar_init(bar(bXC + i), 2);   // [tile][lane quarter]: both half-row warps have published a value
        // [tile][lane quarter][block parity]: the quarter's rescale factors of a block are in shared memory.  One barrier per
        // block parity: the softmax warp may publish block j + 1 before the correction warp has looked at block j, and
        // a single barrier would then be two phases ahead of the waiter.
        for (int i = 0; i < 16; ++i) mbar_init(bar(bAL + i), 1);
        for (int i = 0; i < 4; ++i) mbar_init(bar(bOS + i), 4);   // [tile][P buffer]: the four correction warps are done with O
        mbar_fence_init();
    }
    {
        // delta_s stages: the 256 bytes behind each row stay zero for the whole kernel; ones tile:
        // [k chunk][row group][8 rows][16 bytes], 1.0 in element 0 of every row of chunk 0
        uint4* z = reinterpret_cast<uint4*>(sgen + C::oDelta);
        for (int i = threadIdx.x; i < (S * 2 * C::kDeltaPitch + 4096) / 16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
        if (threadIdx.x < 128) {
            const uint16_t one = std::is_same<OutT, __nv_bfloat16>::value ? 0x3F80 : 0x3C00;
            *reinterpret_cast<uint16_t*>(sgen + C::oOnes + threadIdx.x * 16) = one;
        }
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&tm_q);
        prefetch_tmap(&tm_k);
        prefetch_tmap(&tm_v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const float sl2 = p.sm_scale_per_head ? p.sm_scale_per_head[hq] * 1.4426950408889634f : p.sm_scale_log2;

    // Register budget: 768 threads start with 80 registers each, and that allocation (61 440) is all the CTA can
    // ever hold: 128 x kRoleRegs for warpgroup 0 (three single-lane roles) + 128 x kCorrRegs for the correction
    // warpgroup + 512 x 104 for the softmax warpgroups.  (An increase beyond the launch allocation would wait forever.)
    constexpr int kRoleRegs = (D == 64) ? 24 : 32, kCorrRegs = 64 - kRoleRegs;
    if (warp >= 20) {
      reg_dealloc<kCorrRegs>();
      // ------------------------------------------------------------------ O rescale (correction), one warp per lane quarter
      const int quarter = warp & 3;
      const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
      const float* alpha_s = reinterpret_cast<const float*>(sgen + C::oAlpha);
      const bool carry_in = (p.carry_o_in != nullptr);
      bool ok = true;
      for (int jj = 0; ok && jj < nbmax; ++jj) {
          for (int t = 0; t < 2; ++t) {
              if (jj < skip[t]) continue;
              const int j = jj - skip[t], pb = t * 2 + (j & 1);
              if (!warp_wait(bar(bAL + (t * 4 + quarter) * 2 + (j & 1)), (j >> 1) & 1, abort_flag, p.status, kWaitAlpha)) { ok = false; break; }
              const float alpha = alpha_s[((j & 1) * 2 + t) * 128 + quarter * 32 + lane];
              // block 0 has nothing to rescale unless the accumulator was carried in
              if ((j > 0 || carry_in) && __any_sync(0xffffffffu, alpha != 1.0f)) {
                  // the P V MMA of block j - 1 must have landed first
                  if (j > 0 && !warp_wait(bar(bPV + (pb ^ 1)), ((j - 1) >> 1) & 1, abort_flag, p.status, kWaitOReady)) { ok = false; break; }
                  tc_fence_after();
                  const uint64_t a2 = pack2f(alpha, alpha);
                  const uint32_t o_addr = tmem + lane_addr + C::cO + t * 128;
#pragma unroll
                  for (int cc = 0; cc < D / 16; ++cc) {
                      float o0[16];
                      tmem_ld16(o_addr + cc * 16, o0);
                      tc_wait_ld();
#pragma unroll
                      for (int i = 0; i < 8; ++i)
                          unpack2f(mul2(pack2f(o0[2 * i], o0[2 * i + 1]), a2), o0[2 * i], o0[2 * i + 1]);
                      tmem_st16(o_addr + cc * 16, o0);
                  }
                  tc_wait_st();
              }
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar(bOS + pb));
          }
      }
      __syncwarp();
    } else if (warp < 4) {
      reg_dealloc<kRoleRegs>();
      if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && nbmax > 0) {
            mbar_expect_tx(bar(bQ), nv * (C::kQBytes + C::kSfQkBytes));
            const uint16_t* dptr[2];
            for (int t = 0; t < nv; ++t) {
                tma_load_3d(sbase + C::oQ + t * 8192, &tm_q, bar(bQ), 0, (mt0 + t) * kBlock, bhq);
                bulk_load(sbase + C::oSfQ + t * 1024, p.q_sf + ((size_t)bhq * p.nqt + mt0 + t) * C::kSfQkBytes,
                          C::kSfQkBytes, bar(bQ));
                const int drow = (p.nqm > 1) ? mt0 + t : 0;
                dptr[t] = p.delta + ((size_t)bhq * p.nqm + drow) * ((size_t)p.nkb * kBlock);
            }
            for (int jj = 0; jj < nbmax; ++jj) {
                const int n = nbmax - 1 - jj, st = jj % S;
                if (jj >= S && !mbar_wait<true>(bar(bKE + st), ((jj / S) - 1) & 1, abort_flag, p.status, kWaitKEmpty)) break;
                mbar_expect_tx(bar(bKF + st), C::kKBytes + C::kSfQkBytes + nv * C::kDeltaBytes);
                tma_load_3d(sbase + C::oK + st * 8192, &tm_k, bar(bKF + st), 0, n * kBlock, bhkv);
                bulk_load(sbase + C::oSfK + st * 1024, p.k_sf + ((size_t)bhkv * p.nkb + n) * C::kSfQkBytes,
                          C::kSfQkBytes, bar(bKF + st));
                for (int t = 0; t < nv; ++t)
                    bulk_load(sbase + C::oDelta + (st * 2 + t) * C::kDeltaPitch, dptr[t] + (size_t)n * kBlock,
                              C::kDeltaBytes, bar(bKF + st));
                if (jj >= S && !mbar_wait<true>(bar(bVE + st), ((jj / S) - 1) & 1, abort_flag, p.status, kWaitVEmpty)) break;
                mbar_expect_tx(bar(bVF + st), C::kVBytes + C::kSfVBytes);
                tma_load_3d(sbase + C::oV + st * 8192, &tm_v, bar(bVF + st), n * 64, 0, bhkv);
                bulk_load(sbase + C::oSfV + st * 1024, p.v_sf + ((size_t)bhkv * p.nkb + n) * C::kSfVBytes,
                          C::kSfVBytes, bar(bVF + st));
            }
        }
        __syncwarp();
      } else if (warp == 1) {
        // ------------------------------------------------------------------ Q K^T MMA issuer
        // The single S buffer is handed from tile to tile: it is free again as soon as the four warps of the
        // tile that owned it hold the scores in registers.
        if (lane == 0 && nbmax > 0) {
            constexpr uint32_t idesc_qk = make_idesc_nvfp4(128);
            constexpr uint32_t idesc_delta = make_idesc_f16_bmn(128, std::is_same<OutT, __nv_bfloat16>::value);
            const uint64_t ones_desc = make_sdesc(sbase + C::oOnes, 2048, 128, kSwzNone);
            bool ok = mbar_wait(bar(bQ), 0, abort_flag, p.status, kWaitQFull);
            if (ok) {
                for (int t = 0; t < nv; ++t)
#pragma unroll
                    for (int ks = 0; ks < D / 64; ++ks)
                        tc_cp_sf(tmem + C::cSfQ + 8 * t + 4 * ks, make_sdesc(sbase + C::oSfQ + t * 1024 + ks * 512, 0, 128, kSwzNone));
            }
            int uses = 0;
            for (int jj = 0; ok && jj < nbmax; ++jj) {
                const int st = jj % S;
                if (!mbar_wait(bar(bKF + st), (jj / S) & 1, abort_flag, p.status, kWaitKFull)) { ok = false; break; }
                TR(16, jj, 8)
                tc_fence_after();
                const uint64_t k_desc = make_sdesc(sbase + C::oK + st * 8192, 16, C::kSboQK, C::kSwzQK);
#pragma unroll
                for (int ks = 0; ks < D / 64; ++ks)
                    tc_cp_sf(tmem + C::cSfK + 4 * ks, make_sdesc(sbase + C::oSfK + st * 1024 + ks * 512, 0, 128, kSwzNone));
                for (int t = 0; t < 2; ++t) {
                    if (jj < skip[t]) continue;
                    if (uses > 0 && !mbar_wait(bar(bSE), (uses - 1) & 1, abort_flag, p.status, kWaitSEmpty)) { ok = false; break; }
                    TR(16, jj, 4 * t)
                    tc_fence_after();
                    const uint64_t q_desc = make_sdesc(sbase + C::oQ + t * 8192, 16, C::kSboQK, C::kSwzQK);
                    // S <- 1 (x) delta_s: A = [128 x 16] with ones in column 0 (K-major), B = the delta_s row read as an
                    // MN-major [16 x 128] operand whose rows 1..15 alias finite data and meet zeros in A
                    tc_mma_f16(tmem + C::cS, ones_desc,
                               make_sdesc(sbase + C::oDelta + (st * 2 + t) * C::kDeltaPitch, 16, 16, kSwzNone), idesc_delta, false);
#pragma unroll
                    for (int ks = 0; ks < D / 64; ++ks)
                        tc_mma_nvfp4(tmem + C::cS, q_desc + 2 * ks, k_desc + 2 * ks, idesc_qk,
                                     tmem + C::cSfQ + 8 * t + 4 * ks, tmem + C::cSfK + 4 * ks, true);
                    tc_commit(bar(bSF + t));
                    TR(16, jj, 4 * t + 1)
                    ++uses;
                }
                if (ok) tc_commit(bar(bKE + st));
            }
        }
        __syncwarp();
      } else if (warp == 2) {
        // ------------------------------------------------------------------ PV MMA issuer
        if (lane == 0 && nbmax > 0) {
            constexpr uint32_t idesc_pv = make_idesc_nvfp4(D);
            bool ok = true;
            for (int jj = 0; ok && jj < nbmax; ++jj) {
                const int st = jj % S;
                if (!mbar_wait(bar(bVF + st), (jj / S) & 1, abort_flag, p.status, kWaitVFull)) break;
                TR(17, jj, 8)
                const uint64_t v_desc = make_sdesc(sbase + C::oV + st * 8192, 16, 512, kSwz64);
                bool first = true;
                for (int t = 0; t < 2; ++t) {
                    if (jj < skip[t]) continue;
                    const int j = jj - skip[t], pb = t * 2 + (j & 1);
                    if (!mbar_wait(bar(bPF + pb), (j >> 1) & 1, abort_flag, p.status, kWaitPFull)) { ok = false; break; }
                    if (!mbar_wait(bar(bOS + pb), (j >> 1) & 1, abort_flag, p.status, kWaitOScaled)) { ok = false; break; }
                    TR(17, jj, 4 * t)
                    tc_fence_after();
                    if (first) {
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks)
                            tc_cp_sf(tmem + C::cSfV + 4 * ks, make_sdesc(sbase + C::oSfV + st * 1024 + ks * 512, 0, 128, kSwzNone));
                        first = false;
                    }
                    const uint64_t p_desc = make_sdesc(sbase + C::oP + pb * C::kPBytes, 16, 512, kSwz64);
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks)
                        tc_cp_sf(tmem + C::cSfP + 4 * ks, make_sdesc(sbase + C::oSfP + pb * 1024 + ks * 512, 0, 128, kSwzNone));
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks)
                        tc_mma_nvfp4(tmem + C::cO + t * 128, p_desc + 2 * ks, v_desc + 2 * ks, idesc_pv, tmem + C::cSfP + 4 * ks,
                                     tmem + C::cSfV + 4 * ks, (j > 0) || (ks > 0) || (p.carry_o_in != nullptr));
                    tc_commit(bar(bPV + pb));
                    TR(17, jj, 4 * t + 1)
                }
                if (ok) tc_commit(bar(bVE + st));
            }
        }
        __syncwarp();
      }   // warp 3: no role (it completes warpgroup 0 so that it can give its registers away)
    } else {
        reg_alloc<104>();
        // ------------------------------------------------------------------ softmax warpgroups (4 x 4 warps)
        // Warpgroups 2 t and 2 t + 1 own query tile t; a row is shared by two threads (same lane quarter, one in
        // each warpgroup): thread `h` handles keys [64 h, 64 h + 64) of every block and columns [D/2 h, D/2 (h+1))
        // of the O row.  The two exchange the maximum of their halves once per block; everything else (exp2
        // pass, codes and scales of P, partial row sum, O rescale) is private.  Four such warps share a
        // scheduler, so the exp2 unit finds work while others load, reduce or store.
        const int wg = (warp >> 2) - 1;
        const int t = wg >> 1, h = wg & 1;
        const int quarter = warp & 3;            // tensor-memory lane quarter this warp may touch
        const int r = quarter * 32 + lane;       // row inside the tile
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const int mt = mt0 + t;
        const int nb = nbt[t];
        const int grow = mt * kBlock + r;        // query index
        const uint32_t s_addr = tmem + lane_addr + C::cS + 64 * h;
        const uint32_t o_addr = tmem + lane_addr + C::cO + t * 128 + (D / 2) * h;
        const int sw = (r >> 1) & 3;
        const uint64_t sl2x2 = pack2f(sl2, sl2);
        DEV_DUMP(const bool dbg = (p.debug != nullptr && blockIdx.x == 0 && t == 0);)
        float* xch_mine = reinterpret_cast<float*>(sgen + C::oXch) + (t * 2 + h) * 128 + r;
        const float* xch_other = reinterpret_cast<float*>(sgen + C::oXch) + (t * 2 + (h ^ 1)) * 128 + r;
        const uint32_t bar_x = bar(bXC + t * 4 + quarter);
        int xphase = 0;
        float m_run = -INFINITY, l_run = 0.f;
        bool alive = true;
        const bool carry_in = (p.carry_o_in != nullptr);
        const size_t crow = (size_t)bhq * p.Nq + grow;           // row of the carried state
        if (carry_in && t < nv && !dead_launch) {
            // resume: the accumulator continues from the state an earlier call left (its key range came later in the walk)
            const bool live = grow < Nq;
            m_run = live ? p.carry_m_in[crow] : -INFINITY;
            l_run = live ? p.carry_l_in[2 * crow + h] : 0.f;          // each of the row's two threads keeps its own partial sum
            if (nb > 0) {
#pragma unroll
                for (int cc = 0; cc < D / 64; ++cc) {
                    float o[32];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 v4 = live ? *reinterpret_cast<const float4*>(p.carry_o_in + crow * D + (D / 2) * h + cc * 32 + 4 * i)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
                        o[4 * i] = v4.x; o[4 * i + 1] = v4.y; o[4 * i + 2] = v4.z; o[4 * i + 3] = v4.w;
                    }
                    tmem_st32(o_addr + cc * 32, o);
                }
                tc_wait_st();
                // The correction warp rescales whole rows at block 0, and only thread 0 of a row hands the factors
                // over: the partner's stores have to be ordered before that hand-over.
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_x);
                alive = warp_wait(bar_x, xphase, abort_flag, p.status, kWaitPair);
                xphase ^= 1;
                tc_fence_after();
            }
        }
        PT_DECL
        for (int j = 0; alive && j < nb; ++j) {
            const int n = nb - 1 - j, pb = t * 2 + (j & 1);
            TR(warp - 4, j, 0)
            if (!warp_wait(bar(bSF + t), j & 1, abort_flag, p.status, kWaitSFull)) { alive = false; break; }
            TR(warp - 4, j, 1)
            PT(0)
            tc_fence_after();
            float s[64];
            tmem_ld32(s_addr, s);
            tmem_ld32(s_addr + 32, s + 32);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bSE));     // S is in registers: the other tile's Q K^T may overwrite it
            TR(warp - 4, j, 2)
            PT(1)
            const bool need_mask = ((n + 1) * kBlock > Nk) || (CAUSAL && (n * kBlock + kBlock - 1 > mt * kBlock + shift));
            if (need_mask) {
                int lim = Nk - 1;
                if (CAUSAL) lim = min(lim, grow + shift);
                const int key0 = n * kBlock + 64 * h;
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (key0 + i > lim) s[i] = -INFINITY;
            }
            DEV_DUMP(if (dbg && j == 0) {
                for (int i = 0; i < 64; ++i) p.debug[r * 128 + 64 * h + i] = s[i];
            })
            // Microblock maxima interleaved with the exp2 pass: E = P~ / sf = 6 * 2^((S - bm) s) of a microblock needs only that
            // microblock's maximum, so the maxima of microblock g + 1 are found while the exponentials of microblock g are
            // in flight; the half maximum goes to the partner thread as soon as the last microblock maximum is known (the
            // partner reads it after its own pass).
            float bm[4];
            uint32_t codes[8];
            float se[4];
            float m_half = -INFINITY;
            auto mb_max = [&](int g) {
                const float* x = s + 16 * g;
                float a = fmax3(x[0], x[1], x[2]);
                float b = fmax3(x[3], x[4], x[5]);
                const float c = fmax3(x[6], x[7], x[8]);
                const float d = fmax3(x[9], x[10], x[11]);
                a = fmax3(a, x[12], x[13]);
                b = fmax3(b, x[14], x[15]);
                bm[g] = fmax3(a, b, fmaxf(c, d));
            };
            mb_max(0);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const float negc = (bm[g] == -INFINITY) ? 0.f : -fmaf(bm[g], sl2, -kLog2Of6);
                const uint64_t negc2 = pack2f(negc, negc);
                float e[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a, b2;
                    unpack2f(fma2(pack2f(s[16 * g + 2 * i], s[16 * g + 2 * i + 1]), sl2x2, negc2), a, b2);
                    e[2 * i] = ex2_approx(a);
                    e[2 * i + 1] = ex2_approx(b2);
                }
                if (g < 3) mb_max(g + 1);
                if (g == 2) {
                    m_half = fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3]));
                    xch_mine[(j & 1) * 512] = m_half;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_x);
                    TR(warp - 4, j, 3)
                    PT(2)
                }
                uint64_t acc0 = pack2f(e[0], e[1]), acc1 = pack2f(e[2], e[3]);
                acc0 = add2(acc0, pack2f(e[4], e[5]));
                acc1 = add2(acc1, pack2f(e[6], e[7]));
                acc0 = add2(acc0, pack2f(e[8], e[9]));
                acc1 = add2(acc1, pack2f(e[10], e[11]));
                acc0 = add2(acc0, pack2f(e[12], e[13]));
                acc1 = add2(acc1, pack2f(e[14], e[15]));
                float se0, se1;
                unpack2f(add2(acc0, acc1), se0, se1);
                se[g] = se0 + se1;
                codes[2 * g] = cvt_e2m1x8(e[0], e[1], e[2], e[3], e[4], e[5], e[6], e[7]);
                codes[2 * g + 1] = cvt_e2m1x8(e[8], e[9], e[10], e[11], e[12], e[13], e[14], e[15]);
            }
            TR(warp - 4, j, 4)
            PT(3)
            // running maximum (with the partner's half, published before its own exp2 pass), rescale factor,
            // E4M3 scale sf = max(P~) / 6 = 2^(bm s - max_scaled - log2 6) of every microblock, weighted sum
            if (!warp_wait(bar_x, xphase, abort_flag, p.status, kWaitPair)) { alive = false; break; }
            xphase ^= 1;
            TR(warp - 4, j, 5)
            const float m_new = fmax3(m_run, m_half, xch_other[(j & 1) * 512]);
            const bool empty = (m_new == -INFINITY);
            const float m_cur = empty ? 0.f : m_new;
            const float alpha = ex2_approx((m_run - m_cur) * sl2);        // m_run = -inf  ->  0
            const float max_scaled = empty ? 0.f : fmaf(m_new, sl2, kPScaleLog2);
            m_run = m_new;
            DEV_DUMP(if (dbg && j == 0 && h == 0) p.debug[16384 + r] = m_new;)
            uint32_t sfb = 0;
            float rowsum = 0.f;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const float sfv = (bm[g] == -INFINITY) ? 0.f : ex2_approx(fmaf(bm[g], sl2, -max_scaled) - kLog2Of6);
                rowsum = fmaf(sfv, se[g], rowsum);
                sfb |= (cvt_e4m3x2(sfv, 0.f) & 0xffu) << (8 * g);
            }
            l_run = fmaf(l_run, alpha, rowsum);      // partial row sum of this thread's keys
            DEV_DUMP(if (dbg && j == 0) p.debug[16384 + 128 + 128 * h + r] = rowsum;)
            // P buffer j & 1 was last read by the PV MMA of block j - 2
            if (j >= 2 && !warp_wait(bar(bPV + pb), ((j >> 1) - 1) & 1, abort_flag, p.status, kWaitPEmpty)) { alive = false; break; }
            TR(warp - 4, j, 6)
            PT(4)
            // rescale factors to the correction warp of this lane quarter (slot j & 1 was last read for block j - 2, whose
            // P V MMA has completed, and that MMA is issued only after the correction warp is done)
            if (h == 0) {
                reinterpret_cast<float*>(sgen + C::oAlpha)[((j & 1) * 2 + t) * 128 + r] = alpha;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(bAL + (t * 4 + quarter) * 2 + (j & 1)));
            }
            // P codes: this half's two 16-byte chunks of the 64-byte-swizzled K-major row; scales: its 64-key atom
            uint8_t* prow = sgen + C::oP + pb * C::kPBytes + r * 64;
            uint32_t* sfp_row = reinterpret_cast<uint32_t*>(sgen + C::oSfP + pb * 1024 + (r & 31) * 16 + (r >> 5) * 4);
#pragma unroll
            for (int c = 0; c < 2; ++c)
                *reinterpret_cast<uint4*>(prow + (((2 * h + c) ^ sw) << 4)) =
                    make_uint4(codes[4 * c], codes[4 * c + 1], codes[4 * c + 2], codes[4 * c + 3]);
            sfp_row[128 * h] = sfb;
            fence_proxy_async_smem();
            TR(warp - 4, j, 7)
            PT(5)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bPF + pb));
            TR(warp - 4, j, 9)
            PT(6)
        }
        PT_DUMP(warp)
        // ------------------------------------------------------------------ epilogue: O / l
        if (alive && !dead_launch && t < nv) {
            // the row sum is the sum of the two threads' partial sums (both refer to the same running maximum)
            float* lx = reinterpret_cast<float*>(sgen + C::oXch) + 8 * 128;
            lx[(t * 2 + h) * 128 + r] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_x);
            alive = warp_wait(bar_x, xphase, abort_flag, p.status, kWaitPair);
            const float l_tot = l_run + lx[(t * 2 + (h ^ 1)) * 128 + r];
            if (alive && nb > 0) {
                alive = warp_wait(bar(bPV + t * 2 + ((nb - 1) & 1)), ((nb - 1) >> 1) & 1, abort_flag, p.status, kWaitOReady);
                tc_fence_after();
            }
            if (alive && p.lse != nullptr && h == 0 && grow < Nq) {
                // ln sum_k exp(scale * q.k): the kernel's row sum is 2688 * sum_k 2^((S_k - m) s) over the smoothed
                // scores S (delta_s included); K smoothing took scale * q.km out of every score of the row
                const float ms_fin = (m_run == -INFINITY ? 0.f : m_run) * sl2;
                const float scale = p.sm_scale_per_head ? p.sm_scale_per_head[hq] : p.sm_scale;
                const float v = (ms_fin + __log2f(l_tot) + kPScaleLog2) * 0.6931471805599453f +
                                scale * p.qkm[(size_t)bhq * p.nqt * kBlock + grow];
                p.lse[(size_t)bhq * p.Nq + grow] = (l_tot == 0.f) ? -INFINITY : v;
            }
            if (alive) {
                const float inv_l = (l_tot == 0.f || l_tot != l_tot) ? 0.f : __frcp_rn(l_tot);
                const bool want_out = (p.out[0] != nullptr);
                // the row's home: one output buffer, or the part that owns this token (another GPU's memory when the
                // output goes straight back to the token shards of a sequence-parallel group: plain stores)
                const int opart = (p.out_rows == 0) ? 0 : min(grow / p.out_rows, kMaxParts - 1);
                const int orow_l = grow - opart * p.out_rows;
                OutT* orow = static_cast<OutT*>(p.out[opart]) + out_base + hq * p.os1 + (int64_t)orow_l * p.os2 + (D / 2) * h;
                if (p.carry_o_out != nullptr && grow < Nq) {
                    if (h == 0) p.carry_m_out[crow] = m_run;
                    p.carry_l_out[2 * crow + h] = l_run;
                }
#pragma unroll
                for (int cc = 0; cc < D / 64; ++cc) {
                    float o[32];
                    if (nb > 0) {
                        tmem_ld32(o_addr + cc * 32, o);
                        tc_wait_ld();
                    } else if (carry_in && grow < Nq) {
                        // no key block of this call is visible to the tile: the state passes through
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 v4 = *reinterpret_cast<const float4*>(p.carry_o_in + crow * D + (D / 2) * h + cc * 32 + 4 * i);
                            o[4 * i] = v4.x; o[4 * i + 1] = v4.y; o[4 * i + 2] = v4.z; o[4 * i + 3] = v4.w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = 0.f;
                    }
                    DEV_DUMP(if (dbg) {
                        for (int i = 0; i < 32; ++i) p.debug[16384 + 512 + r * D + (D / 2) * h + cc * 32 + i] = o[i];
                        if (cc == 0 && h == 0) p.debug[16384 + 384 + r] = l_tot;
                    })
                    if (p.carry_o_out != nullptr && grow < Nq) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<float4*>(p.carry_o_out + crow * D + (D / 2) * h + cc * 32 + 4 * i) =
                                make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                    }
                    if (want_out && grow < Nq) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint4 w;
                            w.x = pack2<OutT>(o[8 * i] * inv_l, o[8 * i + 1] * inv_l);
                            w.y = pack2<OutT>(o[8 * i + 2] * inv_l, o[8 * i + 3] * inv_l);
                            w.z = pack2<OutT>(o[8 * i + 4] * inv_l, o[8 * i + 5] * inv_l);
                            w.w = pack2<OutT>(o[8 * i + 6] * inv_l, o[8 * i + 7] * inv_l);
                            *reinterpret_cast<uint4*>(orow + cc * 32 + i * 8) = w;
                        }
                    }
                }
            }
        }
        __syncwarp();
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0) {
        // a wait gave up: give copies that may still be in flight time to land before the CTA retires
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// ------------------------------------------------------------------------------------------------
// host side: tensor maps + launch
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
    return fn;
}

// byte tensor [n2][n1][n0] (n0 contiguous), box [1][b1][b0]
static CUresult make_map(EncodeTiledFn fn, CUtensorMap* m, const void* base, uint64_t n0, uint64_t n1, uint64_t n2,
                         uint32_t b0, uint32_t b1, CUtensorMapSwizzle swz) {
    cuuint64_t dims[3] = {n0, n1, n2};
    cuuint64_t strides[2] = {n0, n0 * n1};
    cuuint32_t box[3] = {b0, b1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

int encode_tiled_bytes(void* map64, const void* base, uint64_t n0, uint64_t n1, uint64_t n2, uint32_t b0, uint32_t b1, int swizzle) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -1;
    const CUtensorMapSwizzle swz = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                 : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    return (int)make_map(fn, static_cast<CUtensorMap*>(map64), base, n0, n1, n2, b0, b1, swz);
}

template <int D, bool CAUSAL, typename OutT, bool VARLEN>
static cudaError_t launch_v(const AttnArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const AttnParams& p, cudaStream_t st) {
    auto kern = attn_fwd_kernel<D, CAUSAL, OutT, VARLEN>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes);
    if (e != cudaSuccess) return e;
    const int grid = a.B * a.Hq * ((a.Nq_p / kBlock + 1) / 2);      // one CTA per pair of query tiles
    kern<<<grid, Cfg<D>::kThreads, Cfg<D>::kSmemBytes, st>>>(tq, tk, tv, p);
    return cudaGetLastError();
}

template <int D, bool CAUSAL, typename OutT>
static cudaError_t launch_t(const AttnArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const AttnParams& p, cudaStream_t st) {
    // packed variable-length batches run their own instantiation, so that the uniform kernels carry none of it
    return a.cu_q != nullptr ? launch_v<D, CAUSAL, OutT, true>(a, tq, tk, tv, p, st)
                             : launch_v<D, CAUSAL, OutT, false>(a, tq, tk, tv, p, st);
}

cudaError_t launch_attn(const AttnArgs& a, cudaStream_t st, int* driver_rc) {
    *driver_rc = 0;
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return cudaErrorNotSupported;
    CUtensorMap tq, tk, tv;
    const uint32_t rowb = a.D / 2;
    const CUtensorMapSwizzle swz_qk = (a.D == 128) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    CUresult r = make_map(fn, &tq, a.q_codes, rowb, a.Nq_p, (uint64_t)a.B * a.Hq, rowb, kBlock, swz_qk);
    if (r == CUDA_SUCCESS) r = make_map(fn, &tk, a.k_codes, rowb, a.Nk_p, (uint64_t)a.B * a.Hkv, rowb, kBlock, swz_qk);
    if (r == CUDA_SUCCESS)
        r = make_map(fn, &tv, a.v_codes, a.Nk_p / 2, a.D, (uint64_t)a.B * a.Hkv, 64, a.D, CU_TENSOR_MAP_SWIZZLE_64B);
    if (r != CUDA_SUCCESS) {
        *driver_rc = (int)r;
        return cudaErrorInvalidValue;
    }
    AttnParams p;
    p.Hq = a.Hq; p.Hkv = a.Hkv; p.Nq = a.Nq; p.Nk = a.Nk;
    p.nqt = a.Nq_p / kBlock; p.nkb = a.Nk_p / kBlock; p.nqm = a.nqm;
    p.sm_scale_log2 = a.sm_scale * 1.4426950408889634f;
    p.sm_scale_per_head = a.sm_scale_per_head;
    p.q_sf = a.q_sf; p.k_sf = a.k_sf; p.v_sf = a.v_sf;
    p.delta = static_cast<const uint16_t*>(a.delta);
    for (int i = 0; i < kMaxParts; ++i) p.out[i] = a.out.base[i];
    p.out_rows = a.out.rows;
    p.lse = a.lse; p.qkm = a.qkm; p.sm_scale = a.sm_scale;
    p.os0 = a.os[0]; p.os1 = a.os[1]; p.os2 = a.os[2];
    p.status = a.status;
    p.prepass_status = a.prepass_status;
    p.carry_o_in = a.carry_o_in; p.carry_m_in = a.carry_m_in; p.carry_l_in = a.carry_l_in;
    p.carry_o_out = a.carry_o_out; p.carry_m_out = a.carry_m_out; p.carry_l_out = a.carry_l_out;
    p.causal_shift = a.causal_shift;
    p.cu_q = a.cu_q; p.cu_k = a.cu_k;
#ifdef SAGE3_DEV_TRACE
    p.debug = a.debug;
#endif
    if (a.is_bf16) {
        if (a.D == 128) return a.is_causal ? launch_t<128, true, __nv_bfloat16>(a, tq, tk, tv, p, st)
                                           : launch_t<128, false, __nv_bfloat16>(a, tq, tk, tv, p, st);
        return a.is_causal ? launch_t<64, true, __nv_bfloat16>(a, tq, tk, tv, p, st)
                           : launch_t<64, false, __nv_bfloat16>(a, tq, tk, tv, p, st);
    }
    if (a.D == 128) return a.is_causal ? launch_t<128, true, __half>(a, tq, tk, tv, p, st)
                                       : launch_t<128, false, __half>(a, tq, tk, tv, p, st);
    return a.is_causal ? launch_t<64, true, __half>(a, tq, tk, tv, p, st)
                       : launch_t<64, false, __half>(a, tq, tk, tv, p, st);
}

}  // namespace sage3
