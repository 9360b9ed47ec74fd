// Pre-pass kernels: K smoothing, Q smoothing, delta_s = qm . k'^T, and NVFP4 quantization of Q, K and
// V-transposed into the layouts the attention kernel consumes.  HBM-bound; 128-bit loads, staged and
// coalesced stores.
//
// Math follows (paths inside the reference project, sageattention3_blackwell/sageattn3/...):
//   api.py:84            k' = k - mean_N(k)                 (mean: fp32 sum, rounded to the input type)
//   api.py:26-72, 86-90  q' = q - mean of each 128-row block (16-bit additions in the Triton kernel's order) or of all padded rows
//   api.py:91            delta_s = qm . k'^T, rounded to the input type (tcgen05 16-bit MMA, accumulator in TMEM)
//   quantization/fp4_quantization_4d.cu:185-225   SF = e4m3(amax / 6), code = e2m1(x * (1 / SF))
//   quantization/fp4_quantization_4d.cu:300-349   V: microblocks are 16 consecutive tokens of one channel
// Divisions and reciprocals are IEEE (div.rn / rcp.rn) so the result can be checked bit for bit.
#include <mutex>

#include "../../include/sage3_b200.h"
#include <cuda.h>

#include "sage3_common.cuh"
#include "sage3_kernels.h"

namespace sage3 {

template <typename T> struct Num;
template <> struct Num<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static constexpr bool kIsBf16 = true;
    static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
    static __device__ __forceinline__ float2 to_f2(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {     // two values rounded to T, lo in bits 0..15
        const __nv_bfloat162 pr = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&pr);
    }
    // packed pairs: each result rounded once to T, which for sums and differences of two T values equals fp32
    // arithmetic followed by a rounding to T (the fp32 result is exact unless the smaller operand lies below a
    // quarter ulp of the larger, where both roundings return the larger operand)
    static __device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
        const __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
        const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t a) {   // max(m, |a|) per half
        const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&m), __habs2(*reinterpret_cast<const __nv_bfloat162*>(&a)));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
};
template <> struct Num<__half> {
    using T2 = __half2;
    static constexpr bool kIsBf16 = false;
    static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
    static __device__ __forceinline__ float2 to_f2(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
    }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        const __half2 pr = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&pr);
    }
    static __device__ __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
        const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
        const __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
    static __device__ __forceinline__ uint32_t absmax2(uint32_t m, uint32_t a) {
        const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&m), __habs2(*reinterpret_cast<const __half2*>(&a)));
        return *reinterpret_cast<const uint32_t*>(&r);
    }
};

// Rows of an input tensor that may be split over several buffers along the token dimension.
template <typename T>
struct Src {
    const T* part[kMaxParts];
    int rows;                       // tokens per part; 0 = everything in part[0]
    const int* cu;                  // packed variable-length sequences: batch entry b owns rows cu[b] .. cu[b + 1]; nullptr: uniform
    // Element offset of (batch entry b, head h); with `cu` also replaces N (the maximum length) by the entry's own length.
    __device__ __forceinline__ int64_t base(int b, int h, int64_t sb, int64_t sh, int64_t sn, int& N) const {
        if (cu != nullptr) {
            const int r0 = cu[b];
            N = min(max(cu[b + 1] - r0, 0), N);
            return (int64_t)r0 * sn + h * sh;
        }
        return b * sb + h * sh;
    }
    __device__ __forceinline__ const T* row(int64_t bh_off, int r, int64_t sn) const {
        if (rows == 0) return part[0] + bh_off + (int64_t)r * sn;
        const int pi = min(r / rows, kMaxParts - 1);
        return part[pi] + bh_off + (int64_t)(r - pi * rows) * sn;
    }
};
template <typename T>
static Src<T> make_src(const PartsPtr& a, const int* cu = nullptr) {
    Src<T> s;
    for (int i = 0; i < kMaxParts; ++i) s.part[i] = static_cast<const T*>(a.base[i]);
    s.rows = a.rows;
    s.cu = cu;
    return s;
}

// 16 elements stay packed in two 128-bit registers until they are needed (keeps the register count, and with it
// the number of resident CTAs, where an HBM-bound kernel needs it)
template <typename T>
__device__ __forceinline__ void load16_packed(const T* p, bool valid, uint4& a, uint4& b) {
    a = make_uint4(0, 0, 0, 0);
    b = a;
    if (valid) {
        a = __ldg(reinterpret_cast<const uint4*>(p));
        b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    }
}
template <typename T>
__device__ __forceinline__ void unpack16(const uint4& a, const uint4& b, float* f) {   // 16 elements -> fp32
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float2 v = Num<T>::to_f2(w[i]);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

// One NVFP4 microblock: 16 fp32 values (already on the input type's grid) and their maximum magnitude -> 8 bytes of
// codes + scale byte.
__device__ __forceinline__ void quant16_amax(const float* x, float amax, uint32_t& lo, uint32_t& hi, uint32_t& sf_byte) {
    sf_byte = cvt_e4m3x2(__fdiv_rn(amax, 6.0f), 0.f) & 0xffu;
    const float sf = e4m3_to_float(sf_byte);
    const float inv = (sf == 0.f) ? 0.f : __frcp_rn(sf);
    float y[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = __fmul_rn(x[i], inv);
    lo = cvt_e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
    hi = cvt_e2m1x8(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]);
}

// The same from eight packed words of the input type (16 values): the maximum magnitude is found on the packed pairs
// (exact, as fp4_quantization_4d.cu:186-196 does), the scaling runs in fp32.
template <typename T>
__device__ __forceinline__ void quant16_packed(const uint32_t* w, uint32_t& lo, uint32_t& hi, uint32_t& sf_byte) {
    uint32_t m = Num<T>::absmax2(0u, w[0]);
#pragma unroll
    for (int i = 1; i < 8; ++i) m = Num<T>::absmax2(m, w[i]);
    const float2 mm = Num<T>::to_f2(m);
    const float amax = fmaxf(mm.x, mm.y);
    sf_byte = cvt_e4m3x2(__fdiv_rn(amax, 6.0f), 0.f) & 0xffu;
    const float sf = e4m3_to_float(sf_byte);
    const float inv = (sf == 0.f) ? 0.f : __frcp_rn(sf);
    float y[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float2 v = Num<T>::to_f2(w[i]);
        y[2 * i] = __fmul_rn(v.x, inv);
        y[2 * i + 1] = __fmul_rn(v.y, inv);
    }
    lo = cvt_e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
    hi = cvt_e2m1x8(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]);
}

// ------------------------------------------------------------------------------------------------
// column sums over tokens: partial sums per chunk of kRowsPerChunk rows, then a fixed-order finalize
// (deterministic: no atomics, the summation order depends on N only)
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __grid_constant__ Src<T> x, int64_t sb, int64_t sh,
                                                             int64_t sn, int H, int N,
                                                             float* __restrict__ part, int chunks) {   // N: by value, narrowed per entry
    constexpr int TPR = D / 8;           // threads per row (8 elements = 16 bytes each)
    constexpr int RPP = 256 / TPR;       // rows per pass
    const int chunk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int64_t bh_off = x.base(b, h, sb, sh, sn, N);
    const int c8 = threadIdx.x % TPR, rl = threadIdx.x / TPR;
    const int r0 = chunk * kRowsPerChunk;
    const int r1 = min(N, r0 + kRowsPerChunk);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = r0 + rl; r < r1; r += RPP) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(x.row(bh_off, r, sn) + c8 * 8));
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 v = Num<T>::to_f2(w[i]);
            acc[2 * i] += v.x;
            acc[2 * i + 1] += v.y;
        }
    }
    __shared__ float red[RPP][D + 1];
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl][c8 * 8 + i] = acc[i];
    __syncthreads();
    if (threadIdx.x < D) {
        float s = 0.f;
#pragma unroll 4
        for (int i = 0; i < RPP; ++i) s += red[i][threadIdx.x];
        part[((int64_t)bh * chunks + chunk) * D + threadIdx.x] = s;
    }
}

template <typename T, int D>
__global__ void colmean_finalize_kernel(const float* __restrict__ part, int chunks, float inv_count,
                                        T* __restrict__ mean, const int* __restrict__ cu, int H, int pad_to_block) {
    const int bh = blockIdx.x, d = threadIdx.x;
    if (cu != nullptr) {
        // the entry's own token count (rounded up to whole 128-row blocks where the mean is over the padded rows);
        // chunks beyond it hold zeros, so the sum is the one a call on this entry alone would form
        int n = max(cu[bh / H + 1] - cu[bh / H], 0);
        if (pad_to_block) n = (n + kBlock - 1) / kBlock * kBlock;
        inv_count = n > 0 ? 1.0f / (float)n : 0.f;
    }
    float s = 0.f;
    for (int c = 0; c < chunks; ++c) s += part[((int64_t)bh * chunks + c) * D + d];
    mean[(int64_t)bh * D + d] = Num<T>::from_f(s * inv_count);
}

// ------------------------------------------------------------------------------------------------
// Q: smooth + quantize one 128-row tile per CTA
// ------------------------------------------------------------------------------------------------
enum { kModeQBlockMean = 0, kModeQGlobalMean = 1 };

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(256, D == 128 ? 4 : 3) quant_rows_kernel(
    const __grid_constant__ Src<T> x, int64_t sb, int64_t sh, int64_t sn, int H, int N, int Np,
    const T* __restrict__ mean_in,     // one mean per head: qm [B*H][D]; unused for block mean
    T* __restrict__ qm_out,            // block mean: [B*H][Np/128][D]
    uint8_t* __restrict__ codes,       // [B*H][Np][D/2]
    uint8_t* __restrict__ sfs,         // [B*H][Np/128][D/64][512]
    const T* __restrict__ km,          // K means [B*Hkv][D]
    int group,                         // query heads per kv head
    float* __restrict__ qkm) {         // [B*H][Np]: x . km per row (the score part that K smoothing removes)
    constexpr int CH = D / 16;            // microblocks per row
    constexpr int RPP = 256 / CH;         // rows per pass
    constexpr int ITEMS = kBlock / RPP;   // microblocks per thread

    const int tile = blockIdx.x, bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int t = threadIdx.x;
    const int c = t % CH, rl = t / CH;
    const int64_t bh_off = x.base(b, h, sb, sh, sn, N);
    const int row0 = tile * kBlock;
    if (row0 >= N && row0 > 0) return;    // a tile beyond this entry's padded length (variable-length batches only)

    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* s_mean = reinterpret_cast<float*>(smem_raw);                        // [D]
    uint8_t* s_sf = smem_raw + D * 4;                                          // [(D/64) * 512]
    uint8_t* s_more = s_sf + (D / 64) * 512;                                   // block mean only: staged tile, chain sums

    uint4 raw[ITEMS][2];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int r = row0 + rl + RPP * i;
        load16_packed<T>(x.row(bh_off, r, sn) + c * 16, r < N, raw[i][0], raw[i][1]);
    }

    // x . km of every row: 16 products per thread, then a sum over the CH neighbouring lanes that share the row
    {
        const T* kmh = km + ((int64_t)b * (H / group) + h / group) * D + c * 16;
        uint4 k0, k1;
        load16_packed<T>(kmh, true, k0, k1);
        float kf[16];
        unpack16<T>(k0, k1, kf);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            float f[16];
            unpack16<T>(raw[i][0], raw[i][1], f);
            float dot = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) dot = fmaf(f[j], kf[j], dot);
#pragma unroll
            for (int off = 1; off < CH; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
            if (c == 0) qkm[(int64_t)bh * Np + row0 + rl + RPP * i] = dot;
        }
    }

    if (MODE == kModeQBlockMean) {
        // Block mean exactly as the reference's Triton kernel forms it (api.py:45-48): a sum of 16-bit values whose every
        // addition rounds to the input type, in the order of that kernel's 4-warp blocked layout:
        //   chain (w, l): rows rep * R + w * L + l, rep = 0 .. 128 / R - 1, added in order of rep
        //                 (L = 32 / (D / 8) rows of a warp, R = 4 L rows per repetition),
        //   then a butterfly over l inside each warp (distance L/2, L/4, ...), then (w0 + w2) + (w1 + w3).
        // Rows beyond N are zero and take part (padding precedes the mean).  The tile is staged in shared memory so
        // that one thread can walk one chain for four columns.
        constexpr int L = 32 / (D / 8), R = 4 * L, REPS = kBlock / R;
        static_assert(R * (D / 4) == 256, "one thread per (chain, group of four columns)");
        T* s_tile = reinterpret_cast<T*>(s_more);                              // [128][D]
        T* s_part = s_tile + kBlock * D;                                       // [R][D]
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            uint4* dst = reinterpret_cast<uint4*>(s_tile + (rl + RPP * i) * D + c * 16);
            dst[0] = raw[i][0];
            dst[1] = raw[i][1];
        }
        __syncthreads();
        {
            const int chain = t / (D / 4), c4 = (t % (D / 4)) * 4;
            uint2 acc = *reinterpret_cast<const uint2*>(s_tile + chain * D + c4);
#pragma unroll
            for (int rep = 1; rep < REPS; ++rep) {
                const uint2 w1 = *reinterpret_cast<const uint2*>(s_tile + (rep * R + chain) * D + c4);
                acc.x = Num<T>::add2(acc.x, w1.x);
                acc.y = Num<T>::add2(acc.y, w1.y);
            }
            *reinterpret_cast<uint2*>(s_part + chain * D + c4) = acc;
        }
        __syncthreads();
        if (t < D) {
            float v[4][L];
#pragma unroll
            for (int w = 0; w < 4; ++w)
#pragma unroll
                for (int l = 0; l < L; ++l) v[w][l] = Num<T>::to_f(s_part[(w * L + l) * D + t]);
            auto add_t = [](float a, float b) { return Num<T>::to_f(Num<T>::from_f(a + b)); };
            float wsum[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
                for (int n = L / 2; n > 0; n >>= 1) {
                    float nv[L];
#pragma unroll
                    for (int l = 0; l < L; ++l) nv[l] = add_t(v[w][l], v[w][l ^ n]);
#pragma unroll
                    for (int l = 0; l < L; ++l) v[w][l] = nv[l];
                }
                wsum[w] = v[w][0];
            }
            const float tot = add_t(add_t(wsum[0], wsum[2]), add_t(wsum[1], wsum[3]));
            const T m = Num<T>::from_f(tot * (1.0f / kBlock));
            s_mean[t] = Num<T>::to_f(m);
            qm_out[((int64_t)bh * (Np / kBlock) + tile) * D + t] = m;
        }
    } else {
        if (t < D) s_mean[t] = Num<T>::to_f(mean_in[(int64_t)bh * D + t]);
    }
    __syncthreads();

    uint32_t mu2[8];       // the 16 means of this thread's columns, packed (they are values of the input type)
#pragma unroll
    for (int j = 0; j < 8; ++j) mu2[j] = Num<T>::pack2(s_mean[c * 16 + 2 * j], s_mean[c * 16 + 2 * j + 1]);

#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int rt = rl + RPP * i;          // row inside the tile
        const int r = row0 + rt;
        // rows beyond N hold 0 - mean (Q is padded before smoothing); they are never read back
        const uint32_t x2[8] = {raw[i][0].x, raw[i][0].y, raw[i][0].z, raw[i][0].w, raw[i][1].x, raw[i][1].y, raw[i][1].z, raw[i][1].w};
        uint32_t d2[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) d2[j] = Num<T>::sub2(x2[j], mu2[j]);
        uint32_t lo, hi, sfb;
        quant16_packed<T>(d2, lo, hi, sfb);
        *reinterpret_cast<uint2*>(codes + ((int64_t)bh * Np + r) * (D / 2) + c * 8) = make_uint2(lo, hi);
        s_sf[sf_atom_offset(rt, c)] = static_cast<uint8_t>(sfb);
    }
    __syncthreads();
    // scale factors of the tile: (D/64) atoms of 512 bytes, contiguous
    {
        uint8_t* dst = sfs + ((int64_t)bh * (Np / kBlock) + tile) * (D / 64) * 512;
        if (t < (D / 64) * 32) reinterpret_cast<uint4*>(dst)[t] = reinterpret_cast<const uint4*>(s_sf)[t];
    }
}

// ------------------------------------------------------------------------------------------------
// K: smooth + quantize one 128-key tile per CTA, and its delta_s columns on the tensor core:
// delta_s[qb][key] = sum_d qm[qb][d] * k'[key][d] as 128 x 128 x D tcgen05 MMAs (16-bit operands from shared
// memory in the 128-byte-swizzled K-major layout, fp32 accumulator in tensor memory), one per 128 query blocks.
// The query-block means arrive through TMA (a tensor map over qm) and the delta_s tiles leave through TMA (a tensor
// map over delta), so the threads' load / store instructions carry only the K rows, the codes and the staging of
// the converted accumulator.
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256, 3) quant_k_delta_kernel(
    const __grid_constant__ Src<T> x, int64_t sb, int64_t sh, int64_t sn, int H, int N, int Np,
    const T* __restrict__ km,          // [B*H][D]
    uint8_t* __restrict__ codes,       // [B*H][Np][D/2]
    uint8_t* __restrict__ sfs,         // [B*H][Np/128][D/64][512]
    int Hq, int nqm, int* __restrict__ status, const int* __restrict__ cu_q,
    const __grid_constant__ CUtensorMap tm_qm,       // bytes [B*Hq][nqm][2 D], box 128 rows x 128 bytes, 128-byte swizzle
    const __grid_constant__ CUtensorMap tm_delta) {  // bytes [B*Hq][nqm][2 Np], box 32 rows x 128 bytes, 128-byte swizzle
    constexpr int CH = D / 16;            // microblocks per row
    constexpr int RPP = 256 / CH;         // rows per pass
    constexpr int ITEMS = kBlock / RPP;   // microblocks per thread
    constexpr int SUB = D / 64;           // 64-element (128-byte) sub-tiles along K
    constexpr uint32_t kTmemCols = 128;
    constexpr bool kBf16 = sizeof(T) == 2 && Num<T>::kIsBf16;

    const int tile = blockIdx.x, bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int c = t % CH, rl = t / CH;
    const int64_t bh_off = x.base(b, h, sb, sh, sn, N);
    const int row0 = tile * kBlock;
    if (row0 >= N && row0 > 0) return;    // a tile beyond this entry's padded length (variable-length batches only)
    // query blocks this entry really has (nqm stays the row count of the qm / delta_s layouts)
    const int nqm_live = (cu_q != nullptr) ? min(nqm, (max(cu_q[b + 1] - cu_q[b], 0) + kBlock - 1) / kBlock) : nqm;

    extern __shared__ uint8_t smem_dyn[];
    const uint32_t sbase = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* sgen = smem_dyn + (sbase - smem_u32(smem_dyn));
    // [B tile: k' | A tile: qm chunk] as SUB sub-tiles of 128 rows x 128 bytes each, then small things, then (D = 64 only,
    // where the A tile is too small for it) the staging tile of the epilogue: 8 warps x 32 rows x 128 bytes
    constexpr int oB = 0, oA = SUB * 16384, oMean = 2 * SUB * 16384, oSf = oMean + D * 4, oBar = oSf + SUB * 512;
    constexpr int oStg = (D == 128) ? oA : ((oBar + 64 + 1023) / 1024) * 1024;
    float* s_mean = reinterpret_cast<float*>(sgen + oMean);
    uint8_t* s_sf = sgen + oSf;
    const uint32_t bar = sbase + oBar;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + oBar + 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sgen + oBar + 12);

    const uint32_t bar_a = bar + 16;        // "the A tile has landed" (the bytes between hold the abort flag and the tensor-memory slot)
    if (t == 0) {
        *abort_flag = 0;
        mbar_init(bar, 1);
        mbar_init(bar_a, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    uint4 raw[ITEMS][2];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int r = row0 + rl + RPP * i;
        load16_packed<T>(x.row(bh_off, r, sn) + c * 16, r < N, raw[i][0], raw[i][1]);
    }
    if (t < D) s_mean[t] = Num<T>::to_f(km[(int64_t)bh * D + t]);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    uint32_t mu2[8];       // the 16 means of this thread's columns, packed (they are values of the input type)
#pragma unroll
    for (int j = 0; j < 8; ++j) mu2[j] = Num<T>::pack2(s_mean[c * 16 + 2 * j], s_mean[c * 16 + 2 * j + 1]);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int rt = rl + RPP * i;          // row inside the tile
        const int r = row0 + rt;
        const bool zero_row = (r >= N);       // K is padded after smoothing: pad rows are 0
        const uint32_t x2[8] = {raw[i][0].x, raw[i][0].y, raw[i][0].z, raw[i][0].w, raw[i][1].x, raw[i][1].y, raw[i][1].z, raw[i][1].w};
        uint32_t w[8];         // k' of this item, packed: quantized below and stored as the MMA operand as it is
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = zero_row ? 0u : Num<T>::sub2(x2[j], mu2[j]);
        uint32_t lo, hi, sfb;
        quant16_packed<T>(w, lo, hi, sfb);
        *reinterpret_cast<uint2*>(codes + ((int64_t)bh * Np + r) * (D / 2) + c * 8) = make_uint2(lo, hi);
        s_sf[sf_atom_offset(rt, c)] = static_cast<uint8_t>(sfb);
        // k' into the B tile: this item's 16 elements are the 16-byte chunks 2c, 2c+1 of row rt
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
            const int chunk = 2 * c + q2, sub = chunk >> 3, cw = chunk & 7;
            *reinterpret_cast<uint4*>(sgen + oB + sub * 16384 + rt * 128 + ((cw ^ (rt & 7)) << 4)) =
                make_uint4(w[4 * q2], w[4 * q2 + 1], w[4 * q2 + 2], w[4 * q2 + 3]);
        }
    }
    __syncthreads();
    {
        uint8_t* dst = sfs + ((int64_t)bh * (Np / kBlock) + tile) * (D / 64) * 512;
        if (t < (D / 64) * 32) reinterpret_cast<uint4*>(dst)[t] = reinterpret_cast<const uint4*>(s_sf)[t];
    }

    // delta_s for every query head of this kv head, 128 query blocks per MMA group
    constexpr uint32_t idesc = make_idesc_f16_kk(128, kBf16);
    const int group = Hq / H;
    const int quarter = warp & 3, chalf = warp >> 2;       // tensor-memory lane quarter, column half of the epilogue
    uint32_t iter = 0;
    bool alive = true;
    for (int g = 0; g < group && alive; ++g) {
        const int hq = h * group + g;
        for (int m0 = 0; m0 < nqm_live && alive; m0 += 128, ++iter) {
            // A tile: 128 query-block means, fetched by the copy engine in the 128-byte swizzle the MMA reads.  Rows beyond
            // the tensor's nqm arrive as zeros; rows of a shorter sequence of a packed batch only feed accumulator rows
            // that nobody reads.
            fence_proxy_async_smem();       // this thread's stores (the k' tile; the previous epilogue's staging) before the engine touches the tiles
            __syncthreads();
            if (t == 0) {
                mbar_expect_tx(bar_a, SUB * 16384);
#pragma unroll
                for (int sub = 0; sub < SUB; ++sub)
                    tma_load_3d(sbase + oA + sub * 16384, &tm_qm, bar_a, sub * 128, m0, b * Hq + hq);
            }
            alive = mbar_wait(bar_a, iter & 1, abort_flag, status, kWaitDeltaA);
            tc_fence_before();
            alive = __syncthreads_and(alive ? 1 : 0) != 0;
            if (!alive) break;
            if (t == 0) {
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * 16384 + (ks & 3) * 32;
                    tc_mma_f16(tmem, make_sdesc(sbase + oA + off, 16, 1024, kSwz128), make_sdesc(sbase + oB + off, 16, 1024, kSwz128),
                               idesc, ks > 0);
                }
                tc_commit(bar);
            }
            alive = mbar_wait(bar, iter & 1, abort_flag, status, kWaitDeltaMma);
            alive = __syncthreads_and(alive ? 1 : 0) != 0;
            if (!alive) break;
            tc_fence_after();
            // epilogue: thread = query block (row) of the accumulator, 64 keys of its row = 128 contiguous bytes of delta_s.
            // The warp's 32 rows x 128 bytes are staged in shared memory in the 128-byte swizzle (at D = 128 in the A tile,
            // which is free once the MMAs have completed) and leave as one TMA tile store; the engine clips rows beyond nqm.
            {
                const uint32_t acc = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + chalf * 64;
                uint8_t* stg = sgen + oStg + warp * 4096;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    float v[32];
                    tmem_ld32(acc + cc * 32, v);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t p4[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) p4[e] = Num<T>::pack2(v[8 * i + 2 * e], v[8 * i + 2 * e + 1]);
                        *reinterpret_cast<uint4*>(stg + lane * 128 + (((cc * 4 + i) ^ (lane & 7)) << 4)) =
                            make_uint4(p4[0], p4[1], p4[2], p4[3]);
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && m0 + quarter * 32 < nqm) {
                    tma_store_3d(&tm_delta, sbase + oStg + warp * 4096, (row0 + chalf * 64) * 2, m0 + quarter * 32, b * Hq + hq);
                    bulk_commit_group();
                    bulk_wait_group_read0();      // the engine has read the staging tile: it may be written again
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncthreads();      // the accumulator and the A tile are free again
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------
// V: one tile of 128 tokens x D channels per CTA -> V^T codes (microblocks along tokens) + scale atoms
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256, 5) quant_vt_kernel(const __grid_constant__ Src<T> x, int64_t sb, int64_t sh, int64_t sn,
                                                       int H, int N, int Np, uint8_t* __restrict__ codes,
                                                       uint8_t* __restrict__ sfs) {
    constexpr int PITCH = D + 2;          // elements; word pitch odd -> column reads are conflict-free
    const int tile = blockIdx.x, bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int t = threadIdx.x;
    const int64_t bh_off = x.base(b, h, sb, sh, sn, N);
    const int row0 = tile * kBlock;
    if (row0 >= N && row0 > 0) return;    // a tile beyond this entry's padded length (variable-length batches only)

    extern __shared__ __align__(16) uint8_t smem_raw[];
    T* s_v = reinterpret_cast<T*>(smem_raw);                                  // [128][PITCH]
    constexpr int OPITCH = 72;            // bytes per staged output row (64 + 8: 8-byte stores stay conflict-free)
    uint8_t* s_out = smem_raw + ((kBlock * PITCH * 2 + 15) / 16) * 16;          // [D][OPITCH] codes
    uint8_t* s_sf = s_out + D * OPITCH;                                        // [2 * 512]

    // zero the scale atoms (rows >= D of a 128-row atom stay zero)
    if (t < 64) reinterpret_cast<uint4*>(s_sf)[t] = make_uint4(0, 0, 0, 0);
    // coalesced load: 16 bytes per thread per pass
    constexpr int TPR = D / 8, RPP = 256 / TPR;
    for (int r = t / TPR; r < kBlock; r += RPP) {
        const int c8 = t % TPR;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row0 + r < N) val = __ldg(reinterpret_cast<const uint4*>(x.row(bh_off, row0 + r, sn) + c8 * 8));
        uint32_t* dst = reinterpret_cast<uint32_t*>(s_v + r * PITCH + c8 * 8);   // 4-byte aligned (PITCH even)
        dst[0] = val.x; dst[1] = val.y; dst[2] = val.z; dst[3] = val.w;
    }
    __syncthreads();
    // two microblocks per item: (channels 2*dp and 2*dp + 1, token group mb); channel pair fastest across
    // threads, so every shared-memory read is one conflict-free 32-bit word holding both channels
    for (int item = t; item < (D / 2) * 8; item += 256) {
        const int dp = item % (D / 2), mb = item / (D / 2);
        float y0[16], y1[16];
        uint32_t m2 = 0u;           // running maximum magnitude of both channels, packed
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(s_v + (mb * 16 + i) * PITCH + 2 * dp);
            m2 = Num<T>::absmax2(m2, w);
            const float2 v2 = Num<T>::to_f2(w);
            y0[i] = v2.x;
            y1[i] = v2.y;
        }
        const float2 amax2 = Num<T>::to_f2(m2);
        uint32_t lo, hi, sfb;
        quant16_amax(y0, amax2.x, lo, hi, sfb);
        *reinterpret_cast<uint2*>(s_out + (2 * dp) * OPITCH + mb * 8) = make_uint2(lo, hi);
        s_sf[sf_atom_offset(2 * dp, mb)] = static_cast<uint8_t>(sfb);
        quant16_amax(y1, amax2.y, lo, hi, sfb);
        *reinterpret_cast<uint2*>(s_out + (2 * dp + 1) * OPITCH + mb * 8) = make_uint2(lo, hi);
        s_sf[sf_atom_offset(2 * dp + 1, mb)] = static_cast<uint8_t>(sfb);
    }
    __syncthreads();
    // coalesced stores: D rows of 64 bytes
    for (int idx = t; idx < D * 8; idx += 256) {
        const int d = idx >> 3, q = idx & 7;
        *reinterpret_cast<uint2*>(codes + ((int64_t)bh * D + d) * (Np / 2) + tile * 64 + q * 8) =
            *reinterpret_cast<const uint2*>(s_out + d * OPITCH + q * 8);
    }
    if (t < 64) {
        uint8_t* dst = sfs + ((int64_t)bh * (Np / kBlock) + tile) * 1024;
        reinterpret_cast<uint4*>(dst)[t] = reinterpret_cast<const uint4*>(s_sf)[t];
    }
}

// ------------------------------------------------------------------------------------------------
// host-side launch
// ------------------------------------------------------------------------------------------------
template <typename T, int D>
static cudaError_t launch_prepass_t(const PrepassArgs& a, cudaStream_t st) {
    const Src<T> q = make_src<T>(a.q, a.cu_q), k = make_src<T>(a.k, a.cu_k), v = make_src<T>(a.v, a.cu_k);
    T* km = static_cast<T*>(a.km);
    T* qm = static_cast<T*>(a.qm);
    T* delta = static_cast<T*>(a.delta);
    const int BHq = a.B * a.Hq, BHkv = a.B * a.Hkv;

    // K mean over its Nk tokens (unless the caller supplied it, e.g. the mean over all shards of a longer sequence)
    if (!a.km_given) {
        colsum_partial_kernel<T, D><<<dim3(a.kchunks_k, BHkv), 256, 0, st>>>(k, a.ks[0], a.ks[1], a.ks[2], a.Hkv, a.Nk,
                                                                             a.kpart, a.kchunks_k);
        colmean_finalize_kernel<T, D><<<BHkv, D, 0, st>>>(a.kpart, a.kchunks_k, 1.0f / (float)a.Nk, km, a.cu_k, a.Hkv, 0);
    }

    const size_t smem_q = D * 4 + (D / 64) * 512;
    if (a.per_block_mean) {
        // + the staged tile [128][D] and the chain sums [4 * 32 / (D / 8)][D] of the block mean
        const size_t smem_qb = smem_q + (kBlock + 4 * (32 / (D / 8))) * D * sizeof(T);
        quant_rows_kernel<T, D, kModeQBlockMean><<<dim3(a.Nq_p / kBlock, BHq), 256, smem_qb, st>>>(
            q, a.qs[0], a.qs[1], a.qs[2], a.Hq, a.Nq, a.Nq_p, nullptr, qm, a.q_codes, a.q_sf, km, a.Hq / a.Hkv, a.qkm);
    } else {
        // one mean per head over the padded rows (api.py:88-90); kpart is free again: the K finalize has
        // consumed it and stream order serializes the two uses
        colsum_partial_kernel<T, D><<<dim3(a.kchunks_q, BHq), 256, 0, st>>>(q, a.qs[0], a.qs[1], a.qs[2], a.Hq, a.Nq,
                                                                            a.kpart, a.kchunks_q);
        colmean_finalize_kernel<T, D><<<BHq, D, 0, st>>>(a.kpart, a.kchunks_q, 1.0f / (float)a.Nq_p, qm, a.cu_q, a.Hq, 1);
        quant_rows_kernel<T, D, kModeQGlobalMean><<<dim3(a.Nq_p / kBlock, BHq), 256, smem_q, st>>>(
            q, a.qs[0], a.qs[1], a.qs[2], a.Hq, a.Nq, a.Nq_p, qm, nullptr, a.q_codes, a.q_sf, km, a.Hq / a.Hkv, a.qkm);
    }
    const size_t smem_k = 2 * (D / 64) * 16384 + D * 4 + (D / 64) * 512 + 64 + 1024 + (D == 64 ? 1024 + 32768 : 0);
    cudaError_t e = cudaFuncSetAttribute(quant_k_delta_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_k);
    if (e != cudaSuccess) return e;
    // tensor maps for the K kernel: the Q means [B*Hq][nqm][D] and delta_s [B*Hq][nqm][Nk_p] as byte tensors
    alignas(64) CUtensorMap tm_qm, tm_delta;
    if (encode_tiled_bytes(&tm_qm, qm, (uint64_t)D * 2, (uint64_t)a.nqm, (uint64_t)a.B * a.Hq, 128, 128, 3) != 0 ||
        encode_tiled_bytes(&tm_delta, delta, (uint64_t)a.Nk_p * 2, (uint64_t)a.nqm, (uint64_t)a.B * a.Hq, 128, 32, 3) != 0)
        return cudaErrorInvalidValue;
    quant_k_delta_kernel<T, D><<<dim3(a.Nk_p / kBlock, BHkv), 256, smem_k, st>>>(
        k, a.ks[0], a.ks[1], a.ks[2], a.Hkv, a.Nk, a.Nk_p, km, a.k_codes, a.k_sf, a.Hq, a.nqm, a.status, a.cu_q, tm_qm, tm_delta);

    const size_t smem_v = ((kBlock * (D + 2) * sizeof(T) + 15) / 16) * 16 + D * 72 + 1024;
    e = cudaFuncSetAttribute(quant_vt_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_v);
    if (e != cudaSuccess) return e;
    quant_vt_kernel<T, D><<<dim3(a.Nk_p / kBlock, BHkv), 256, smem_v, st>>>(v, a.vs[0], a.vs[1], a.vs[2], a.Hkv, a.Nk,
                                                                           a.Nk_p, a.v_codes, a.v_sf);
    return cudaGetLastError();
}

cudaError_t launch_prepass(const PrepassArgs& a, cudaStream_t st) {
    if (a.is_bf16) {
        return a.D == 128 ? launch_prepass_t<__nv_bfloat16, 128>(a, st) : launch_prepass_t<__nv_bfloat16, 64>(a, st);
    }
    return a.D == 128 ? launch_prepass_t<__half, 128>(a, st) : launch_prepass_t<__half, 64>(a, st);
}

}  // namespace sage3

// ------------------------------------------------------------------------------------------------
// K mean without any allocation by anybody: the partial column sums live in a static device array
// ------------------------------------------------------------------------------------------------
namespace {

// Scratch for sage3_kmean_noalloc: partial column sums [B*Hkv][chunks][D] in fp32.  Every GPU that loads this
// library holds these 4 MiB until the process exits.  Inside host code this name is only a stand-in for the
// device array; the device address is obtained once per device with cudaGetSymbolAddress (below).
static __device__ __align__(256) float g_kmean_scratch[SAGE3_KMEAN_NOALLOC_MAX_FLOATS];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
float* g_scratch_addr[kMaxDevices] = {};   // device address of g_kmean_scratch on each device, once resolved

// Device address of the scratch array on the current device; resolved on the first call per device.
int scratch_for_current_device(float** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return SAGE3_E_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return SAGE3_E_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_kmean_scratch) != cudaSuccess || p == nullptr) return SAGE3_E_CUDA;
        g_scratch_addr[dev] = static_cast<float*>(p);
    }
    *out = g_scratch_addr[dev];
    return SAGE3_OK;
}

template <typename T, int D>
cudaError_t launch_kmean_t(const Sage3Desc* d, const void* k, void* km, float* scratch, int chunks, cudaStream_t st) {
    const int BH = d->B * d->Hkv;
    sage3::PartsPtr one = {};
    one.base[0] = const_cast<void*>(k);
    sage3::colsum_partial_kernel<T, D><<<dim3(chunks, BH), 256, 0, st>>>(
        sage3::make_src<T>(one), d->k_stride[0], d->k_stride[1], d->k_stride[2], d->Hkv, d->Nk, scratch, chunks);
    sage3::colmean_finalize_kernel<T, D><<<BH, D, 0, st>>>(scratch, chunks, 1.0f / (float)d->Nk, static_cast<T*>(km), nullptr, d->Hkv, 0);
    return cudaGetLastError();
}

}  // namespace

// Column means from partial column sums: mean[r][d] = round(dtype, (sum over c, in order, of part[r][c][d]) * (1 / count)).
// The second half of the K-mean stage on its own, for callers that gather the partial sums of several token shards
// (one 512-row chunk after the other, shard after shard) and need the mean the single call forms, bit for bit.
extern "C" SAGE3_API int sage3_mean_from_partial_sums(const float* part, int32_t rows, int32_t chunks, int32_t D, int32_t dtype,
                                                      int64_t count, void* mean_out, void* stream) {
    if (!part || !mean_out) return SAGE3_E_NULL;
    if (rows <= 0 || chunks <= 0 || count <= 0 || (D != 64 && D != 128)) return SAGE3_E_SHAPE;
    if (dtype != SAGE3_FP16 && dtype != SAGE3_BF16) return SAGE3_E_DTYPE;
    if ((reinterpret_cast<uintptr_t>(part) % 4) != 0 || (reinterpret_cast<uintptr_t>(mean_out) % 2) != 0) return SAGE3_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const float inv = 1.0f / (float)count;
    if (dtype == SAGE3_BF16) {
        if (D == 128) sage3::colmean_finalize_kernel<__nv_bfloat16, 128><<<rows, 128, 0, st>>>(part, chunks, inv, static_cast<__nv_bfloat16*>(mean_out), nullptr, 1, 0);
        else sage3::colmean_finalize_kernel<__nv_bfloat16, 64><<<rows, 64, 0, st>>>(part, chunks, inv, static_cast<__nv_bfloat16*>(mean_out), nullptr, 1, 0);
    } else {
        if (D == 128) sage3::colmean_finalize_kernel<__half, 128><<<rows, 128, 0, st>>>(part, chunks, inv, static_cast<__half*>(mean_out), nullptr, 1, 0);
        else sage3::colmean_finalize_kernel<__half, 64><<<rows, 64, 0, st>>>(part, chunks, inv, static_cast<__half*>(mean_out), nullptr, 1, 0);
    }
    return cudaGetLastError() == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

extern "C" SAGE3_API int sage3_kmean_noalloc(const Sage3Desc* desc, const void* k, void* km_out, void* stream) {
    if (!desc || !k || !km_out) return SAGE3_E_NULL;
    if (desc->B <= 0 || desc->Hkv <= 0 || desc->Nk <= 0 || (desc->D != 64 && desc->D != 128)) return SAGE3_E_SHAPE;
    if (desc->dtype != SAGE3_FP16 && desc->dtype != SAGE3_BF16) return SAGE3_E_DTYPE;
    for (int i = 0; i < 3; ++i)
        if (desc->k_stride[i] < 0 || (desc->k_stride[i] % 8) != 0) return SAGE3_E_STRIDE;
    if ((reinterpret_cast<uintptr_t>(k) % 16) != 0 || (reinterpret_cast<uintptr_t>(km_out) % 2) != 0) return SAGE3_E_ALIGN;
    const int64_t chunks = ((int64_t)desc->Nk + sage3::kRowsPerChunk - 1) / sage3::kRowsPerChunk;
    const int64_t need = (int64_t)desc->B * desc->Hkv * chunks * desc->D;
    if (need > (int64_t)SAGE3_KMEAN_NOALLOC_MAX_FLOATS || chunks > 65535) return SAGE3_E_TOO_LARGE;
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess)
        return SAGE3_E_CUDA;
    if (major != 10 || minor != 0) return SAGE3_E_ARCH;
    float* scratch = nullptr;
    const int rc = scratch_for_current_device(&scratch);
    if (rc != SAGE3_OK) return rc;
    // Nothing in the scratch has to start at zero: every partial sum the finalize step reads is written by the
    // first kernel of this very call.
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (desc->dtype == SAGE3_BF16)
        e = desc->D == 128 ? launch_kmean_t<__nv_bfloat16, 128>(desc, k, km_out, scratch, (int)chunks, st)
                           : launch_kmean_t<__nv_bfloat16, 64>(desc, k, km_out, scratch, (int)chunks, st);
    else
        e = desc->D == 128 ? launch_kmean_t<__half, 128>(desc, k, km_out, scratch, (int)chunks, st)
                           : launch_kmean_t<__half, 64>(desc, k, km_out, scratch, (int)chunks, st);
    return e == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}
