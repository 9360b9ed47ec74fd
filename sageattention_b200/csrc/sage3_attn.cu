// Block-scaled FP4 attention for sm_100a: TMA-staged E2M1 tiles, tcgen05 NVFP4 MMAs with the S and O
// accumulators in tensor memory, exp2 online softmax, P re-quantized to NVFP4 before the PV MMA.
//
// One CTA per 128-row query tile.  Ten warps:
//   warp 0      TMA producer (one lane): Q once, then K (+ delta_s row) / V^T / scale atoms per KV block
//   warp 1      MMA issuer (one lane) and owner of the tensor-memory allocation
//   warps 2-9   softmax: thread (row r, column half) owns 64 of the 128 scores of its row per block;
//               the two halves of a row exchange their block maximum through shared memory
// S is double-buffered in tensor memory so that Q K^T of block j+1 overlaps the softmax of block j.
// O stays in tensor memory and is rescaled in place only when a row maximum moved.
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
    static constexpr int oMx = oOnes + 4096;                  // float [2][2][128]
    static constexpr int oBar = oMx + 2 * 2 * 128 * 4;
    static constexpr int kNumBars = 1 + 4 * kStages + 2 + 2 + 2 + 1 + 4;
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
template <typename OutT> __device__ __forceinline__ float delta_to_f(uint32_t h16);
template <> __device__ __forceinline__ float delta_to_f<__nv_bfloat16>(uint32_t h16) { return __uint_as_float(h16 << 16); }
template <> __device__ __forceinline__ float delta_to_f<__half>(uint32_t h16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16)));
}

// Wait executed by a whole converged warp; the verdict is made warp-uniform so that no lane leaves a loop alone.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
    return __all_sync(0xffffffffu, ok);
}

template <int D, bool CAUSAL, typename OutT>
__global__ void __launch_bounds__(320, 1)
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
    const int bQ = 0, bKF = 1, bKE = bKF + S, bVF = bKE + S, bVE = bVF + S, bSF = bVE + S, bSE = bSF + 2,
              bPF = bSE + 2, bOR = bPF + 2, bPair = bOR + 1;
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
            mbar_init(bar(bKE + i), 1);
            mbar_init(bar(bVF + i), 1);
            mbar_init(bar(bVE + i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(bSF + i), 1);
            mbar_init(bar(bSE + i), 8);
            mbar_init(bar(bPF + i), 8);
        }
        mbar_init(bar(bOR), 1);
        for (int i = 0; i < 4; ++i) mbar_init(bar(bPair + i), 2);
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
                if (j >= S && !mbar_wait(bar(bKE + st), ((j / S) - 1) & 1, abort_flag, p.status, kWaitKEmpty)) break;
                mbar_expect_tx(bar(bKF + st), C::kKBytes + C::kSfQkBytes + C::kDeltaBytes);
                tma_load_3d(sbase + C::oK + st * 8192, &tm_k, bar(bKF + st), 0, n * kBlock, bhkv);
                bulk_load(sbase + C::oSfK + st * 1024, p.k_sf + ((size_t)bhkv * p.nkb + n) * C::kSfQkBytes,
                          C::kSfQkBytes, bar(bKF + st));
                bulk_load(sbase + C::oDelta + st * C::kDeltaPitch, dptr + (size_t)n * kBlock, C::kDeltaBytes, bar(bKF + st));
                if (j >= S && !mbar_wait(bar(bVE + st), ((j / S) - 1) & 1, abort_flag, p.status, kWaitVEmpty)) break;
                mbar_expect_tx(bar(bVF + st), C::kVBytes + C::kSfVBytes);
                tma_load_3d(sbase + C::oV + st * 8192, &tm_v, bar(bVF + st), n * 64, 0, bhkv);
                bulk_load(sbase + C::oSfV + st * 1024, p.v_sf + ((size_t)bhkv * p.nkb + n) * C::kSfVBytes,
                          C::kSfVBytes, bar(bVF + st));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && nb > 0) {
            constexpr uint32_t idesc_qk = make_idesc_nvfp4(128);
            constexpr uint32_t idesc_pv = make_idesc_nvfp4(D);
            const uint64_t q_desc = make_sdesc(sbase + C::oQ, 16, C::kSboQK, C::kSwzQK);
            constexpr uint32_t idesc_delta = make_idesc_f16_bmn(128, sizeof(OutT) == 2 && std::is_same<OutT, __nv_bfloat16>::value);
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
                tc_commit(bar(bKE + st));
                tc_commit(bar(bSF + bb));
                return true;
            };
            bool ok = mbar_wait(bar(bQ), 0, abort_flag, p.status, kWaitQFull);
            if (ok) {
#pragma unroll
                for (int ks = 0; ks < D / 64; ++ks)
                    tc_cp_sf(tmem + C::cSfQ + 4 * ks, make_sdesc(sbase + C::oSfQ + ks * 512, 0, 128, kSwzNone));
                ok = issue_qk(0);
            }
            for (int j = 0; ok && j < nb; ++j) {
                const int st = j % S, bb = j & 1;
                if (j + 1 < nb && !issue_qk(j + 1)) break;
                if (!mbar_wait(bar(bVF + st), (j / S) & 1, abort_flag, p.status, kWaitVFull)) break;
                if (!mbar_wait(bar(bPF + bb), (j >> 1) & 1, abort_flag, p.status, kWaitPFull)) break;
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
                tc_commit(bar(bVE + st));
                tc_commit(bar(bOR));
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ softmax + correction + epilogue
        const int quarter = warp & 3;            // tensor-memory lane quarter this warp may touch
        const int half = (warp - 2) >> 2;        // which 64 of the 128 columns
        const int r = quarter * 32 + lane;       // row inside the tile
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        float* s_mx = reinterpret_cast<float*>(sgen + C::oMx);
        const int grow = mt * kBlock + r;        // query index
        float m_run = -INFINITY, l_run = 0.f;
        bool alive = true;

        for (int j = 0; j < nb; ++j) {
            const int n = nb - 1 - j, bb = j & 1;
            if (!warp_wait(bar(bSF + bb), (j >> 1) & 1, abort_flag, p.status, kWaitSFull)) { alive = false; break; }
            tc_fence_after();
            float s[64];
            const uint32_t s_addr = tmem + lane_addr + (bb ? C::cS1 : C::cS0) + half * 64;
            tmem_ld32(s_addr, s);
            tmem_ld32(s_addr + 32, s + 32);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bSE + bb));

            // masks on the real key index: keys beyond Nk, and (causal) keys after the diagonal
            const int key0 = n * kBlock + half * 64;
            const bool need_mask = ((n + 1) * kBlock > p.Nk) || (CAUSAL && (n * kBlock + kBlock - 1 > mt * kBlock + shift));
            if (need_mask) {
                int lim = p.Nk - 1;
                if (CAUSAL) lim = min(lim, grow + shift);
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (key0 + i > lim) s[i] = -INFINITY;
            }
            // microblock maxima and the row maximum of this block
            float bm[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                float a = fmax3(s[16 * g], s[16 * g + 1], s[16 * g + 2]);
#pragma unroll
                for (int i = 3; i < 15; i += 2) a = fmax3(a, s[16 * g + i], s[16 * g + i + 1]);
                bm[g] = fmaxf(a, s[16 * g + 15]);
            }
            const float lmax = fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3]));
            s_mx[(bb * 2 + half) * 128 + r] = lmax;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bPair + quarter));
            if (!warp_wait(bar(bPair + quarter), j & 1, abort_flag, p.status, kWaitPair)) { alive = false; break; }
            __syncwarp();
            const float omax = s_mx[(bb * 2 + (half ^ 1)) * 128 + r];
            const float m_new = fmax3(m_run, lmax, omax);
            const bool empty = (m_new == -INFINITY);
            const float m_cur = empty ? 0.f : m_new;
            const float alpha = ex2_approx((m_run - m_cur) * sl2);
            const float max_scaled = empty ? 0.f : fmaf(m_new, sl2, kPScaleLog2);

            uint32_t codes[8];
            uint32_t sfbytes = 0;
            float rowsum = 0.f;
            const uint64_t sl2x2 = pack2f(sl2, sl2);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const bool gdead = (bm[g] == -INFINITY);
                // E = P~ / sf = 6 * 2^((S - bm) s);   sf = max(P~) / 6 = 2^(bm s - max_scaled - log2 6)
                const float c = gdead ? 0.f : fmaf(bm[g], sl2, -kLog2Of6);
                const float sf = gdead ? 0.f : ex2_approx(fmaf(bm[g], sl2, -max_scaled) - kLog2Of6);
                const uint64_t negc = pack2f(-c, -c);
                float e[16];
                uint64_t acc0 = 0, acc1 = 0;      // two packed partial sums (bit pattern of +0.0f pairs)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a, b2;
                    unpack2f(fma2(pack2f(s[16 * g + 2 * i], s[16 * g + 2 * i + 1]), sl2x2, negc), a, b2);
                    e[2 * i] = ex2_approx(a);
                    e[2 * i + 1] = ex2_approx(b2);
                    if (i & 1) acc1 = add2(acc1, pack2f(e[2 * i], e[2 * i + 1]));
                    else acc0 = add2(acc0, pack2f(e[2 * i], e[2 * i + 1]));
                }
                float se0, se1;
                unpack2f(add2(acc0, acc1), se0, se1);
                rowsum = fmaf(sf, se0 + se1, rowsum);
                codes[2 * g] = cvt_e2m1x8(e[0], e[1], e[2], e[3], e[4], e[5], e[6], e[7]);
                codes[2 * g + 1] = cvt_e2m1x8(e[8], e[9], e[10], e[11], e[12], e[13], e[14], e[15]);
                sfbytes |= (cvt_e4m3x2(sf, 0.f) & 0xffu) << (8 * g);
            }
            l_run = fmaf(l_run, alpha, rowsum);

            // P codes into the 64-byte-swizzled K-major tile; scales into the 128x4 atom of this column half
            {
                uint8_t* prow = sgen + C::oP + bb * C::kPBytes + r * 64;
                const int sw = (r >> 1) & 3;
                *reinterpret_cast<uint4*>(prow + (((2 * half) ^ sw) << 4)) = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                *reinterpret_cast<uint4*>(prow + (((2 * half + 1) ^ sw) << 4)) = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                *reinterpret_cast<uint32_t*>(sgen + C::oSfP + bb * 1024 + half * 512 + (r & 31) * 16 + (r >> 5) * 4) = sfbytes;
            }
            if (p.debug != nullptr && blockIdx.x == 0 && j == 0) {
#pragma unroll
                for (int i = 0; i < 64; ++i) p.debug[r * 128 + half * 64 + i] = s[i];
                if (half == 0) { p.debug[16384 + r] = m_new; }
                p.debug[16384 + 128 + half * 128 + r] = rowsum;
            }
            // O of the previous block must be complete before it is rescaled / before P of block j-2 is reused
            if (j > 0) {
                if (!warp_wait(bar(bOR), (j - 1) & 1, abort_flag, p.status, kWaitOReady)) { alive = false; break; }
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    tc_fence_after();
#pragma unroll
                    for (int cc = 0; cc < D / 64; ++cc) {
                        float o[32];
                        const uint32_t o_addr = tmem + lane_addr + C::cO + half * (D / 2) + cc * 32;
                        tmem_ld32(o_addr, o);
                        tc_wait_ld();
                        const uint64_t a2 = pack2f(alpha, alpha);
#pragma unroll
                        for (int i = 0; i < 16; ++i) unpack2f(mul2(pack2f(o[2 * i], o[2 * i + 1]), a2), o[2 * i], o[2 * i + 1]);
                        tmem_st32(o_addr, o);
                    }
                    tc_wait_st();
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(bPF + bb));
            m_run = m_new;
        }

        // ------------------------------------------------------------------ epilogue
        if (alive && !dead_launch) {
            float l_tot = 0.f;
            if (nb > 0) {
                alive = warp_wait(bar(bOR), (nb - 1) & 1, abort_flag, p.status, kWaitOReady);
                if (alive) {
                    tc_fence_after();
                    const int bb = nb & 1;
                    s_mx[(bb * 2 + half) * 128 + r] = l_run;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(bPair + quarter));
                    alive = warp_wait(bar(bPair + quarter), nb & 1, abort_flag, p.status, kWaitPair);
                    __syncwarp();
                    if (alive) l_tot = l_run + s_mx[(bb * 2 + (half ^ 1)) * 128 + r];
                }
            }
            if (alive) {
                const float inv_l = (l_tot == 0.f || l_tot != l_tot) ? 0.f : __frcp_rn(l_tot);
                OutT* orow = static_cast<OutT*>(p.out) + b * p.os0 + hq * p.os1 + (int64_t)grow * p.os2 + half * (D / 2);
#pragma unroll
                for (int cc = 0; cc < D / 64; ++cc) {
                    float o[32];
                    if (nb > 0) {
                        tmem_ld32(tmem + lane_addr + C::cO + half * (D / 2) + cc * 32, o);
                        tc_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = 0.f;
                    }
                    if (p.debug != nullptr && blockIdx.x == 0) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) p.debug[16384 + 512 + r * D + half * (D / 2) + cc * 32 + i] = o[i];
                        if (half == 0 && cc == 0) p.debug[16384 + 384 + r] = l_tot;
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
    kern<<<grid, 320, Cfg<D>::kSmemBytes, st>>>(tq, tk, tv, p);
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
