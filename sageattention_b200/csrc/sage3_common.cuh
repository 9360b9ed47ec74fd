// Device-side building blocks for the sm_100a kernels: mbarrier, TMA, tcgen05 (MMA / TMEM) wrappers,
// UMMA descriptors and the NVFP4 number formats.  Raw PTX; no CUTLASS / CuTe.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sage3 {

constexpr int kBlock = 128;   // query-tile rows and keys per KV block
constexpr int kMicro = 16;    // NVFP4 microblock

// status-word codes written by device code when a bounded wait gives up
enum : int {
    kWaitQFull = 101, kWaitKFull = 102, kWaitVFull = 103, kWaitKEmpty = 104, kWaitVEmpty = 105,
    kWaitSFull = 106, kWaitSEmpty = 107, kWaitPFull = 108, kWaitOReady = 109, kWaitPair = 110,
    kWaitPEmpty = 113, kWaitAlpha = 114, kWaitOScaled = 112, kWaitDeltaMma = 116, kWaitDeltaA = 117, kWaitSelfTest = 199
};

// ------------------------------------------------------------------------------------------------
// small helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// per-warpgroup register budget (all four warps of a warpgroup execute the same call)
template <int N> __device__ __forceinline__ void reg_alloc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_dealloc() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// packed fp32 pairs (one issue slot for two lanes of math)
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2f(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// ------------------------------------------------------------------------------------------------
// number formats
// ------------------------------------------------------------------------------------------------
// Two fp32 -> one byte of two E2M1 codes; `lo` lands in bits 0-3, `hi` in bits 4-7.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint32_t r;
    asm("{\n\t.reg .b8 b;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b, %2, %1;\n\t"
        "cvt.u32.u8 %0, b;\n\t}"
        : "=r"(r) : "f"(lo), "f"(hi));
    return r;
}

// Eight fp32 -> 32 bits of E2M1 codes, element i in nibble i.
__device__ __forceinline__ uint32_t cvt_e2m1x8(float f0, float f1, float f2, float f3, float f4, float f5,
                                               float f6, float f7) {
    uint32_t r;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(r) : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
    return r;
}

// Two non-negative fp32 -> two E4M3 bytes (lo in bits 0-7), round to nearest even, saturate at 448.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
    return r;
}

// E4M3 byte -> fp32 (exact).
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
    uint32_t h2;
    asm("{\n\t.reg .b16 s;\n\t"
        "cvt.u16.u32 s, %1;\n\t"
        "cvt.rn.f16x2.e4m3x2 %0, s;\n\t}"
        : "=r"(h2) : "r"(b & 0xffu));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

// ------------------------------------------------------------------------------------------------
// mbarrier
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Gives up after `kWaitLimitCycles` SM cycles, or as soon as another thread of the
// CTA (abort flag in shared memory) or another CTA (status word in global memory) has given up.
// On giving up it records `code` in the status word, raises the CTA's abort flag and returns false;
// the caller must then leave its loop.  Nothing ever spins without a limit.
constexpr long long kWaitLimitCycles = 2000000000LL;   // about a second

// kBackoff: sleep a little between polls (single-lane roles, so that polling does not take issue slots
// from the math warps of the same scheduler).
template <bool kBackoff = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, int code, long long limit_cycles = kWaitLimitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (kBackoff) __nanosleep(40);
        if ((++spins & 0x3f) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > limit_cycles || *reinterpret_cast<volatile int*>(status_word) != 0) {
                atomicCAS(status_word, 0, code);
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// TMA (bulk tensor copies; no multicast anywhere)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
// shared -> global tile store (bulk group); the issuing thread commits the group and, before the shared-memory tile is
// written again, waits until the engine has read it
__device__ __forceinline__ void tma_store_3d(const void* tmap, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(tmap), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// contiguous global -> shared copy; src, dst 16-byte aligned, bytes % 16 == 0
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
// make generic-proxy shared-memory writes visible to the async proxy (TMA, tcgen05)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------
// tcgen05: tensor memory and MMA
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {                               // whole warp
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {    // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// all previously issued tcgen05.mma / tcgen05.cp of this thread -> one arrival on `bar` when they finish
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 128 bit of shared memory -> TMEM, replicated into the four 32-lane quarters: one
// 128-row x 4-scale atom of scale factors becomes 4 TMEM columns.
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], NVFP4: E2M1 operands, one UE4M3 scale per 16 elements, K = 64.
__device__ __forceinline__ void tc_mma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], 16-bit operands (fp16 or bf16), fp32 accumulate, K = 16.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
}

// instruction descriptor of the 16-bit MMA: M = 128, N = n, fp32 accumulator, A K-major, B MN-major.
//   bits 4-5: D format (1 = F32), 7-9 / 10-12: A / B format (0 = F16, 1 = BF16), bit 15 / 16: A / B major
//   (0 = K, 1 = MN), bits 17-22: N >> 3, bits 24-28: M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_f16_bmn(int n, bool bf16) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (1u << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

// same, both operands K-major
__host__ __device__ constexpr uint32_t make_idesc_f16_kk(int n, bool bf16) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

// instruction descriptor of the block-scaled NVFP4 MMA: M = 128, N = n, both operands K-major.
//   bits 7-9 / 10-12: A / B format (1 = E2M1), bits 17-22: N >> 3, bit 23: scale format (0 = UE4M3),
//   bits 24-28: M >> 4, bits 4-5 / 29-30: scale-factor byte ids (0), bit 31: K size (0 = 64).
__host__ __device__ constexpr uint32_t make_idesc_nvfp4(int n) {
    return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
}

// shared-memory matrix descriptor, K-major operand.
//   bits 0-13 start address >> 4, 16-29 leading byte offset >> 4, 32-45 stride byte offset >> 4
//   (distance between 8-row groups), 46-47 descriptor version (1 on sm_100), 61-63 swizzle mode.
enum : uint64_t { kSwzNone = 0, kSwz128 = 2, kSwz64 = 4, kSwz32 = 6 };
__device__ __forceinline__ uint64_t make_sdesc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t swz) {
    return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
           (static_cast<uint64_t>(sbo_bytes >> 4) << 32) | (1ull << 46) | (swz << 61);
}

// 32 lanes x 32 columns of 32-bit TMEM cells -> 32 registers per thread (thread i reads lane base+i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]),
          "r"(taddr) : "memory");
}

// byte offset of scale (row r, scale column c) inside a group of 128-row x 4-scale atoms
__host__ __device__ constexpr uint32_t sf_atom_offset(uint32_t r, uint32_t c) {
    return (c >> 2) * 512u + (r & 31u) * 16u + ((r >> 5) & 3u) * 4u + (c & 3u);
}

}  // namespace sage3
