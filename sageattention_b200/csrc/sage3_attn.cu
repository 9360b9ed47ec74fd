// Block-scaled FP4 attention for sm_100a: TMA-staged E2M1 tiles, tcgen05 NVFP4 MMAs with the S and O
// accumulators in tensor memory, exp2 online softmax, P re-quantized to NVFP4 before the PV MMA.
//
// One CTA per 128-row query tile.  Four warpgroups (setmaxnreg moves registers to the exp warpgroups):
//   warp 0       TMA producer (one lane): Q once, then K (+ delta_s row) / V^T / scale atoms per KV block
//   warp 1       Q K^T MMA issuer (one lane) and owner of the tensor-memory allocation
//   warp 2       P V MMA issuer (one lane); warp 3 idle
//   warps 4-11   exp: two warpgroups that take alternate KV blocks; thread = row with all 128 scores of the block
//                in registers -> exp2 values, their row sum and FP4 codes of P; bound by the exp2 unit
//   warps 12-15  stats + correction: thread = row; one block ahead of the exp warps it reads the whole S row,
//                derives microblock maxima, running maximum, rescale factor and per-microblock constants
//                (shared memory -> exp warps), rescales O in tensor memory when a row maximum moved, and
//                finally writes O / l to global memory
// S is double-buffered in tensor memory so that Q K^T and the statistics of block j+1 overlap the exp2 work
// of block j.
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

// Optional per-phase cycle accounting of the first CTA (development builds only; off in the product library).
#ifdef SAGE3_PHASE_TIMING
#define PT_DECL long long pt_t = clock64(); long long pt_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define PT(i) { const long long pt_now = clock64(); pt_acc[i] += pt_now - pt_t; pt_t = pt_now; }
#define PT_DUMP(slot) if (p.debug != nullptr && blockIdx.x == 0 && lane == 0) { for (int i_ = 0; i_ < 8; ++i_) p.debug[40000 + (slot) * 8 + i_] = (float)pt_acc[i_]; }
#else
#define PT_DECL
#define PT(i)
#define PT_DUMP(slot)
#endif

constexpr float kLog2Of6 = 2.584962500721156f;
constexpr float kPScaleLog2 = -11.392317422778762f;   // log2(1 / (448 * 6)), softmax_fused.h:33

struct AttnParams {
    int Hq, Hkv, Nq, Nk, nqt, nkb, nqm;   // nqt = query tiles per head, nkb = KV blocks per head
    float sm_scale_log2;
    const float* sm_scale_per_head;
    const uint8_t *q_sf, *k_sf, *v_sf;
    const uint16_t* delta;              // 16-bit elements [B*Hq][nqm][nkb*128]
    void* out;
    int64_t os0, os1, os2;
    int* status;
    float* debug;                       // optional dump of CTA 0 (nullptr in normal use)
};

template <int D>
struct Cfg {
    static constexpr int kStages = (D == 128) ? 6 : 8;
    static constexpr int kThreads = 512;                      // 4 warpgroups, see the kernel
    static constexpr int kQBytes = 128 * D / 2;
    static constexpr int kSfQkBytes = (D / 64) * 512;
    static constexpr int kKBytes = 128 * D / 2;
    static constexpr int kVBytes = D * 64;
    static constexpr int kSfVBytes = 1024;
    static constexpr int kDeltaBytes = 256;
    static constexpr int kPBytes = 8192;
    static constexpr int kSfPBytes = 1024;
    // shared-memory map (bytes from a 1024-aligned base)
    static constexpr int oQ = 0;
    static constexpr int oK = oQ + 8192;
    static constexpr int oV = oK + kStages * 8192;
    static constexpr int oP = oV + kStages * 8192;
    static constexpr int oSfQ = oP + 2 * kPBytes;
    static constexpr int oSfK = oSfQ + 1024;
    static constexpr int oSfV = oSfK + kStages * 1024;
    static constexpr int oSfP = oSfV + kStages * 1024;
    static constexpr int oDelta = oSfP + 2 * 1024;
    static constexpr int kDeltaPitch = 512;                   // 256 B of delta_s + 256 B that stay zero
    static constexpr int oOnes = oDelta + kStages * kDeltaPitch;   // 128 x 16 tile: column 0 = 1.0, rest 0
    static constexpr int oCst = oOnes + 4096;                 // float [2][17][128]  per block: 8 offsets, 8 scales, scaled max per row
    static constexpr int oL = oCst + 2 * 17 * 128 * 4;        // float [2][2][128]   per exp warpgroup: row sum, scaled max it refers to
    static constexpr int oBar = oL + 4 * 128 * 4;
    static constexpr int kNumBars = 1 + 4 * kStages + 2 + 2 + 1 + 2 + 1;
    static constexpr int oMisc = oBar + kNumBars * 8;
    static constexpr int kSmemBytes = oMisc + 64 + 1024;      // + slack for the manual 1024-byte alignment
    // tensor-memory columns
    static constexpr uint32_t cS0 = 0, cS1 = 128, cO = 256, cSfQ = 384, cSfK = 392, cSfP = 400, cSfV = 408;
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

// Maxima of two 16-key microblocks held in t[0..31] (3-input max: 8 operations per 16 values, depth 3).
__device__ __forceinline__ void microblock_max2(const float* t, float& m0, float& m1) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const float* x = t + 16 * g;
        float a = fmax3(x[0], x[1], x[2]);
        float b = fmax3(x[3], x[4], x[5]);
        const float c = fmax3(x[6], x[7], x[8]);
        const float d = fmax3(x[9], x[10], x[11]);
        a = fmax3(a, x[12], x[13]);
        b = fmax3(b, x[14], x[15]);
        (g ? m1 : m0) = fmax3(a, b, fmaxf(c, d));
    }
}

template <int D, bool CAUSAL, typename OutT>
__global__ void __launch_bounds__(Cfg<D>::kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
    using C = Cfg<D>;
    constexpr int S = C::kStages;
    extern __shared__ uint8_t smem_dyn[];
    const uint32_t sbase = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* sgen = smem_dyn + (sbase - smem_u32(smem_dyn));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // barriers
    auto bar = [&](int i) { return sbase + C::oBar + 8u * i; };
    const int bQ = 0, bKF = 1, bQK = bKF + S, bVF = bQK + S, bPV = bVF + S, bSE = bPV + S, bPF = bSE + 2,
              bOS = bPF + 2, bST = bOS + 1, bLR = bST + 2;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + C::oMisc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + C::oMisc + 8);

    // tile -> (batch*head, query tile); heavier causal tiles are scheduled first
    const int bhq = blockIdx.x / p.nqt;
    int mt = blockIdx.x % p.nqt;
    if (CAUSAL) mt = p.nqt - 1 - mt;
    const int b = bhq / p.Hq, hq = bhq % p.Hq;
    const int bhkv = b * p.Hkv + hq / (p.Hq / p.Hkv);
    const int shift = p.Nk - p.Nq;
    int nb = p.nkb;
    if (CAUSAL) {
        const int max_key = min(p.Nk - 1, mt * kBlock + kBlock - 1 + shift);
        nb = max_key < 0 ? 0 : max_key / kBlock + 1;
    }
    const bool dead_launch = (*reinterpret_cast<volatile int*>(p.status) != 0);   // an earlier CTA gave up
    if (dead_launch) nb = 0;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        mbar_init(bar(bQ), 1);
        for (int i = 0; i < S; ++i) {
            mbar_init(bar(bKF + i), 1);
            mbar_init(bar(bQK + i), 1);    // Q K^T (+ delta_s) of the block in stage i is complete: its S buffer is full, the K stage is free
            mbar_init(bar(bVF + i), 1);
            mbar_init(bar(bPV + i), 1);    // P V of the block in stage i is complete: O is up to date, V stage and P buffer are free
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(bSE + i), 8);    // the exp warpgroup of the block (4 warps) and the stats warps (4) have read S buffer i
            mbar_init(bar(bST + i), 4);    // constants of the block in S buffer i are in shared memory  (stats warps)
            mbar_init(bar(bPF + i), 4);    // P buffer i (+ its scales) is written
        }
        mbar_init(bar(bOS), 4);            // O has been rescaled for the next PV          (stats warps)
        mbar_init(bar(bLR), 8);            // final row sums of both exp warpgroups are in shared memory
        mbar_fence_init();
    }
    {
        // delta_s stages: the 256 bytes behind each row stay zero for the whole kernel; ones tile:
        // [k chunk][row group][8 rows][16 bytes], 1.0 in element 0 of every row of chunk 0
        uint4* z = reinterpret_cast<uint4*>(sgen + C::oDelta);
        for (int i = threadIdx.x; i < (S * C::kDeltaPitch + 4096) / 16; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
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
    float* s_cst = reinterpret_cast<float*>(sgen + C::oCst);
    float* s_l = reinterpret_cast<float*>(sgen + C::oL);

    // Register budget: 512 threads start with 128 registers each; the exp warpgroups (a whole S row per thread)
    // take what warpgroup 0 (two single-lane roles) and the stats warpgroup do not need.
    if (warp < 4) {
      reg_dealloc<48>();
      if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && nb > 0) {
            mbar_expect_tx(bar(bQ), C::kQBytes + C::kSfQkBytes);
            tma_load_3d(sbase + C::oQ, &tm_q, bar(bQ), 0, mt * kBlock, bhq);
            bulk_load(sbase + C::oSfQ, p.q_sf + ((size_t)bhq * p.nqt + mt) * C::kSfQkBytes, C::kSfQkBytes, bar(bQ));
            const int drow = (p.nqm > 1) ? mt : 0;
            const uint16_t* dptr = p.delta + ((size_t)bhq * p.nqm + drow) * ((size_t)p.nkb * kBlock);
            for (int j = 0; j < nb; ++j) {
                const int n = nb - 1 - j, st = j % S;
                if (j >= S && !mbar_wait<true>(bar(bQK + st), ((j / S) - 1) & 1, abort_flag, p.status, kWaitKEmpty)) break;
                mbar_expect_tx(bar(bKF + st), C::kKBytes + C::kSfQkBytes + C::kDeltaBytes);
                tma_load_3d(sbase + C::oK + st * 8192, &tm_k, bar(bKF + st), 0, n * kBlock, bhkv);
                bulk_load(sbase + C::oSfK + st * 1024, p.k_sf + ((size_t)bhkv * p.nkb + n) * C::kSfQkBytes,
                          C::kSfQkBytes, bar(bKF + st));
                bulk_load(sbase + C::oDelta + st * C::kDeltaPitch, dptr + (size_t)n * kBlock, C::kDeltaBytes, bar(bKF + st));
                if (j >= S && !mbar_wait<true>(bar(bPV + st), ((j / S) - 1) & 1, abort_flag, p.status, kWaitVEmpty)) break;
                mbar_expect_tx(bar(bVF + st), C::kVBytes + C::kSfVBytes);
                tma_load_3d(sbase + C::oV + st * 8192, &tm_v, bar(bVF + st), n * 64, 0, bhkv);
                bulk_load(sbase + C::oSfV + st * 1024, p.v_sf + ((size_t)bhkv * p.nkb + n) * C::kSfVBytes,
                          C::kSfVBytes, bar(bVF + st));
            }
        }
        __syncwarp();
      } else if (warp == 1) {
        // ------------------------------------------------------------------ Q K^T MMA issuer
        if (lane == 0 && nb > 0) {
            constexpr uint32_t idesc_qk = make_idesc_nvfp4(128);
            constexpr uint32_t idesc_delta = make_idesc_f16_bmn(128, std::is_same<OutT, __nv_bfloat16>::value);
            const uint64_t q_desc = make_sdesc(sbase + C::oQ, 16, C::kSboQK, C::kSwzQK);
            const uint64_t ones_desc = make_sdesc(sbase + C::oOnes, 2048, 128, kSwzNone);
            auto issue_qk = [&](int j) -> bool {
                const int st = j % S, bb = j & 1;
                if (j >= 2 && !mbar_wait(bar(bSE + bb), ((j >> 1) - 1) & 1, abort_flag, p.status, kWaitSEmpty)) return false;
                if (!mbar_wait(bar(bKF + st), (j / S) & 1, abort_flag, p.status, kWaitKFull)) return false;
                tc_fence_after();
                const uint64_t k_desc = make_sdesc(sbase + C::oK + st * 8192, 16, C::kSboQK, C::kSwzQK);
#pragma unroll
                for (int ks = 0; ks < D / 64; ++ks)
                    tc_cp_sf(tmem + C::cSfK + 4 * ks, make_sdesc(sbase + C::oSfK + st * 1024 + ks * 512, 0, 128, kSwzNone));
                // S <- 1 (x) delta_s: A = [128 x 16] with ones in column 0 (K-major), B = the delta_s row read as an
                // MN-major [16 x 128] operand whose rows 1..15 alias finite data and meet zeros in A
                tc_mma_f16(tmem + (bb ? C::cS1 : C::cS0), ones_desc,
                           make_sdesc(sbase + C::oDelta + st * C::kDeltaPitch, 16, 16, kSwzNone), idesc_delta, false);
#pragma unroll
                for (int ks = 0; ks < D / 64; ++ks)
                    tc_mma_nvfp4(tmem + (bb ? C::cS1 : C::cS0), q_desc + 2 * ks, k_desc + 2 * ks, idesc_qk,
                                 tmem + C::cSfQ + 4 * ks, tmem + C::cSfK + 4 * ks, true);
                tc_commit(bar(bQK + st));
                return true;
            };
            PT_DECL
            bool ok = mbar_wait(bar(bQ), 0, abort_flag, p.status, kWaitQFull);
            if (ok) {
#pragma unroll
                for (int ks = 0; ks < D / 64; ++ks)
                    tc_cp_sf(tmem + C::cSfQ + 4 * ks, make_sdesc(sbase + C::oSfQ + ks * 512, 0, 128, kSwzNone));
            }
            // S buffer j & 1 is free as soon as block j - 2 sits in the registers of its exp and stats warps
            for (int j = 0; ok && j < nb; ++j) {
                ok = issue_qk(j);
                PT(0)
            }
            PT_DUMP(1)
        }
        __syncwarp();
      } else if (warp == 2) {
        // ------------------------------------------------------------------ PV MMA issuer
        if (lane == 0 && nb > 0) {
            constexpr uint32_t idesc_pv = make_idesc_nvfp4(D);
            PT_DECL
            for (int j = 0; j < nb; ++j) {
                const int st = j % S, bb = j & 1;
                if (!mbar_wait(bar(bVF + st), (j / S) & 1, abort_flag, p.status, kWaitVFull)) break;
                PT(1)
                if (!mbar_wait(bar(bPF + bb), (j >> 1) & 1, abort_flag, p.status, kWaitPFull)) break;
                PT(2)
                if (!mbar_wait(bar(bOS), j & 1, abort_flag, p.status, kWaitOScaled)) break;
                PT(3)
                tc_fence_after();
                const uint64_t p_desc = make_sdesc(sbase + C::oP + bb * C::kPBytes, 16, 512, kSwz64);
                const uint64_t v_desc = make_sdesc(sbase + C::oV + st * 8192, 16, 512, kSwz64);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) {
                    tc_cp_sf(tmem + C::cSfP + 4 * ks, make_sdesc(sbase + C::oSfP + bb * 1024 + ks * 512, 0, 128, kSwzNone));
                    tc_cp_sf(tmem + C::cSfV + 4 * ks, make_sdesc(sbase + C::oSfV + st * 1024 + ks * 512, 0, 128, kSwzNone));
                }
#pragma unroll
                for (int ks = 0; ks < 2; ++ks)
                    tc_mma_nvfp4(tmem + C::cO, p_desc + 2 * ks, v_desc + 2 * ks, idesc_pv, tmem + C::cSfP + 4 * ks,
                                 tmem + C::cSfV + 4 * ks, (j > 0) || (ks > 0));
                tc_commit(bar(bPV + st));
                PT(4)
            }
            PT_DUMP(2)
        }
        __syncwarp();
      }   // warp 3: no role (it completes warpgroup 0 so that it can give its registers away)
    } else if (warp < 12) {
        reg_alloc<184>();
        // ------------------------------------------------------------------ exp warpgroups (2 x 4 warps)
        // Warpgroup `par` handles the blocks j = par, par + 2, ...; thread = row r with all 128 scores of the
        // block in registers.  The block's constants (per-microblock offsets and scales, scaled running
        // maximum) come from the stats warps through shared memory; their arrival also tells that S(j) is
        // complete.  The two warpgroups are never
        // synchronised with each other: the loads, waits and stores of one overlap the exp2 work of the other.
        const int quarter = warp & 3;            // tensor-memory lane quarter this warp may touch
        const int par = (warp >> 2) - 1;         // block parity; also the S buffer and the P buffer it uses
        const int r = quarter * 32 + lane;       // row inside the tile
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const int grow = mt * kBlock + r;        // query index
        const uint32_t s_addr = tmem + lane_addr + (par ? C::cS1 : C::cS0);
        const float* cst = s_cst + par * (17 * 128) + r;
        uint8_t* prow = sgen + C::oP + par * C::kPBytes + r * 64;
        uint32_t* sfp_row = reinterpret_cast<uint32_t*>(sgen + C::oSfP + par * 1024 + (r & 31) * 16 + (r >> 5) * 4);
        const int sw = (r >> 1) & 3;
        const uint64_t sl2x2 = pack2f(sl2, sl2);
        float l_run = 0.f, ms_prev = -INFINITY;
        bool alive = true;
        PT_DECL
        for (int j = par; j < nb; j += 2) {
            const int n = nb - 1 - j;
            if (!warp_wait(bar(bST + par), (j >> 1) & 1, abort_flag, p.status, kWaitStats)) { alive = false; break; }
            tc_fence_after();
            float s[128];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) tmem_ld32(s_addr + c4 * 32, s + c4 * 32);
            float negc[8], sfv[8];
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                negc[g] = cst[g * 128];
                sfv[g] = cst[(8 + g) * 128];
            }
            const float ms = cst[16 * 128];
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bSE + par));     // S(j) is in registers, its constants are read
            PT(4)
            const bool need_mask = ((n + 1) * kBlock > p.Nk) || (CAUSAL && (n * kBlock + kBlock - 1 > mt * kBlock + shift));
            if (need_mask) {
                int lim = p.Nk - 1;
                if (CAUSAL) lim = min(lim, grow + shift);
                const int key0 = n * kBlock;
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (key0 + i > lim) s[i] = -INFINITY;
            }
            if (p.debug != nullptr && blockIdx.x == 0 && j == 0) {
#pragma unroll
                for (int i = 0; i < 128; ++i) p.debug[r * 128 + i] = s[i];
            }
            uint32_t codes[16];
            uint32_t sfb[2] = {0, 0};
            float rowsum = 0.f;
            // Software pipeline over the eight microblocks: the exp2 instructions of microblock g + 1 are issued
            // before the sums / conversions of microblock g, so the exp2 unit always has work queued.
            // E = P~ / sf = 6 * 2^((S - bm) s)  with  negc = -(bm s - log2 6)
            float e[16];
            {
                const uint64_t negc2 = pack2f(negc[0], negc[0]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a, b2;
                    unpack2f(fma2(pack2f(s[2 * i], s[2 * i + 1]), sl2x2, negc2), a, b2);
                    e[2 * i] = ex2_approx(a);
                    e[2 * i + 1] = ex2_approx(b2);
                }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                float en[16];
                if (g < 7) {
                    const uint64_t negc2 = pack2f(negc[g + 1], negc[g + 1]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float a, b2;
                        unpack2f(fma2(pack2f(s[16 * (g + 1) + 2 * i], s[16 * (g + 1) + 2 * i + 1]), sl2x2, negc2), a, b2);
                        en[2 * i] = ex2_approx(a);
                        en[2 * i + 1] = ex2_approx(b2);
                    }
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
                rowsum = fmaf(sfv[g], se0 + se1, rowsum);
                codes[2 * g] = cvt_e2m1x8(e[0], e[1], e[2], e[3], e[4], e[5], e[6], e[7]);
                codes[2 * g + 1] = cvt_e2m1x8(e[8], e[9], e[10], e[11], e[12], e[13], e[14], e[15]);
                sfb[g >> 2] |= (cvt_e4m3x2(sfv[g], 0.f) & 0xffu) << (8 * (g & 3));
                if (g < 7) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) e[i] = en[i];
                }
            }
            // row sum relative to the running maximum of this block: rescale what this warpgroup has so far
            const float a_eff = (l_run == 0.f) ? 0.f : ex2_approx(ms_prev - ms);
            l_run = fmaf(l_run, a_eff, rowsum);
            ms_prev = ms;
            if (p.debug != nullptr && blockIdx.x == 0 && j == 0) p.debug[16384 + 128 + r] = rowsum;
            PT(0)
            // P buffer `par` was last read by the PV MMA of block j - 2
            if (j >= 2 && !warp_wait(bar(bPV + (j - 2) % S), ((j - 2) / S) & 1, abort_flag, p.status, kWaitPEmpty)) { alive = false; break; }
            // P codes: four 16-byte chunks of the 64-byte-swizzled K-major row; scales: one word per 64-key atom
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(prow + ((c ^ sw) << 4)) =
                    make_uint4(codes[4 * c], codes[4 * c + 1], codes[4 * c + 2], codes[4 * c + 3]);
            sfp_row[0] = sfb[0];
            sfp_row[128] = sfb[1];
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bPF + par));
            PT(3)
        }
        PT_DUMP(warp)
        // hand the row sum (and the scaled maximum it refers to) to the stats warps
        if (alive && nb > 0) {
            s_l[par * 256 + r] = l_run;
            s_l[par * 256 + 128 + r] = ms_prev;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bLR));
        }
        __syncwarp();
    } else {
        reg_dealloc<96>();
        // ------------------------------------------------------------------ stats + correction + epilogue (4 warps)
        // Thread = row r.  For every block, ahead of the exp warps: microblock maxima of the whole row, running
        // maximum, rescale factor and the per-microblock constants, published through shared memory.  Then O is
        // multiplied by the rescale factor before the block's PV MMA (only when some row of the warp moved its
        // maximum).  At the end O / l goes to global memory.
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const int grow = mt * kBlock + r;
        float m_run = -INFINITY;
        bool alive = true;
        PT_DECL
        // statistics of block j: constants into shared memory, rescale factor returned
        auto do_stats = [&](int j, float& alpha_out) -> bool {
            const int n = nb - 1 - j, bb = j & 1;
            if (!warp_wait(bar(bQK + j % S), (j / S) & 1, abort_flag, p.status, kWaitSFull)) return false;
            PT(0)
            tc_fence_after();
            const bool need_mask = ((n + 1) * kBlock > p.Nk) || (CAUSAL && (n * kBlock + kBlock - 1 > mt * kBlock + shift));
            int lim = p.Nk - 1;
            if (CAUSAL) lim = min(lim, grow + shift);
            auto mask32 = [&](float* t, int c4) {
                const int key0 = n * kBlock + c4 * 32;
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (key0 + i > lim) t[i] = -INFINITY;
            };
            const uint32_t sa = tmem + lane_addr + (bb ? C::cS1 : C::cS0);
            float bm[8];
            float t0[32], t1[32];
            // two loads in flight at a time
            tmem_ld32(sa, t0);
            tmem_ld32(sa + 32, t1);
            tc_wait_ld();
            if (need_mask) { mask32(t0, 0); mask32(t1, 1); }
            microblock_max2(t0, bm[0], bm[1]);
            microblock_max2(t1, bm[2], bm[3]);
            tmem_ld32(sa + 64, t0);
            tmem_ld32(sa + 96, t1);
            tc_wait_ld();
            if (need_mask) { mask32(t0, 2); mask32(t1, 3); }
            microblock_max2(t0, bm[4], bm[5]);
            microblock_max2(t1, bm[6], bm[7]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bSE + bb));
            PT(1)
            const float m_new = fmaxf(fmax3(m_run, bm[0], bm[1]), fmaxf(fmax3(bm[2], bm[3], bm[4]), fmax3(bm[5], bm[6], bm[7])));
            const bool empty = (m_new == -INFINITY);
            const float m_cur = empty ? 0.f : m_new;
            alpha_out = ex2_approx((m_run - m_cur) * sl2);        // m_run = -inf  ->  0
            const float max_scaled = empty ? 0.f : fmaf(m_new, sl2, kPScaleLog2);
            float* cst = s_cst + bb * (17 * 128);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const bool gdead = (bm[g] == -INFINITY);
                // sf = max(P~) / 6 = 2^(bm s - max_scaled - log2 6);  negc = -(bm s - log2 6)
                cst[g * 128 + r] = gdead ? 0.f : -fmaf(bm[g], sl2, -kLog2Of6);
                cst[(8 + g) * 128 + r] = gdead ? 0.f : ex2_approx(fmaf(bm[g], sl2, -max_scaled) - kLog2Of6);
            }
            cst[16 * 128 + r] = m_cur * sl2;      // scaled running maximum the exp2 values of this block refer to
            m_run = m_new;
            if (p.debug != nullptr && blockIdx.x == 0 && j == 0) p.debug[16384 + r] = m_new;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bST + bb));
            PT(2)
            return true;
        };
        float alpha = 1.f;
        if (nb > 0) alive = do_stats(0, alpha);
        for (int j = 0; alive && j < nb; ++j) {
            // statistics run one block ahead of the rescaling, so the exp warps never wait for a PV MMA
            float alpha_next = 1.f;
            if (j + 1 < nb && !do_stats(j + 1, alpha_next)) { alive = false; break; }
            if (j > 0) {
                if (!warp_wait(bar(bPV + (j - 1) % S), ((j - 1) / S) & 1, abort_flag, p.status, kWaitOReady)) { alive = false; break; }
                PT(3)
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    tc_fence_after();
                    const uint64_t a2 = pack2f(alpha, alpha);
#pragma unroll
                    for (int cc = 0; cc < D / 64; ++cc) {
                        float o0[32], o1[32];
                        const uint32_t o_addr = tmem + lane_addr + C::cO + cc * 64;
                        tmem_ld32(o_addr, o0);
                        tmem_ld32(o_addr + 32, o1);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            unpack2f(mul2(pack2f(o0[2 * i], o0[2 * i + 1]), a2), o0[2 * i], o0[2 * i + 1]);
                            unpack2f(mul2(pack2f(o1[2 * i], o1[2 * i + 1]), a2), o1[2 * i], o1[2 * i + 1]);
                        }
                        tmem_st32(o_addr, o0);
                        tmem_st32(o_addr + 32, o1);
                    }
                    tc_wait_st();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bOS));
            alpha = alpha_next;
            PT(4)
        }
        PT_DUMP(warp)
        if (alive && !dead_launch) {
            float l_tot = 0.f;
            if (nb > 0) {
                alive = warp_wait(bar(bLR), 0, abort_flag, p.status, kWaitAlpha);
                if (alive) alive = warp_wait(bar(bPV + (nb - 1) % S), ((nb - 1) / S) & 1, abort_flag, p.status, kWaitOReady);
                if (alive) {
                    tc_fence_after();
                    // each exp warpgroup's sum refers to the maximum of its own last block: bring both to the final one
                    const float ms_final = (m_run == -INFINITY ? 0.f : m_run) * sl2;
#pragma unroll
                    for (int w2 = 0; w2 < 2; ++w2) {
                        const float lw = s_l[w2 * 256 + r], lm = s_l[w2 * 256 + 128 + r];
                        if (lw != 0.f) l_tot += lw * ex2_approx(lm - ms_final);
                    }
                }
            }
            if (alive) {
                const float inv_l = (l_tot == 0.f || l_tot != l_tot) ? 0.f : __frcp_rn(l_tot);
                OutT* orow = static_cast<OutT*>(p.out) + b * p.os0 + hq * p.os1 + (int64_t)grow * p.os2;
#pragma unroll
                for (int cc = 0; cc < D / 32; ++cc) {
                    float o[32];
                    if (nb > 0) {
                        tmem_ld32(tmem + lane_addr + C::cO + cc * 32, o);
                        tc_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = 0.f;
                    }
                    if (p.debug != nullptr && blockIdx.x == 0) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) p.debug[16384 + 512 + r * D + cc * 32 + i] = o[i];
                        if (cc == 0) p.debug[16384 + 384 + r] = l_tot;
                    }
                    if (grow < p.Nq) {
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

template <int D, bool CAUSAL, typename OutT>
static cudaError_t launch_t(const AttnArgs& a, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const AttnParams& p, cudaStream_t st) {
    auto kern = attn_fwd_kernel<D, CAUSAL, OutT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<D>::kSmemBytes);
    if (e != cudaSuccess) return e;
    const int grid = a.B * a.Hq * (a.Nq_p / kBlock);
    kern<<<grid, Cfg<D>::kThreads, Cfg<D>::kSmemBytes, st>>>(tq, tk, tv, p);
    return cudaGetLastError();
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
    p.out = a.out;
    p.os0 = a.os[0]; p.os1 = a.os[1]; p.os2 = a.os[2];
    p.status = a.status;
    p.debug = a.debug;
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
