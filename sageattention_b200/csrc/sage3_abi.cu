// extern "C" boundary of libsage3_b200.so (declared in include/sage3_b200.h): argument validation,
// workspace layout, and the launches.  No allocation, no caching of caller pointers, no exceptions.
#include <cuda_runtime.h>
#include <string.h>

#include "../../include/sage3_b200.h"
#include "sage3_common.cuh"
#include "sage3_kernels.h"

namespace {

constexpr size_t kAlign = 1024;     // every workspace region starts at a multiple of this from the base
constexpr size_t kWsAlign = 256;    // required alignment of the workspace base pointer
inline size_t align_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

int validate(const Sage3Desc* d) {
    if (!d) return SAGE3_E_NULL;
    if (d->B <= 0 || d->Hq <= 0 || d->Hkv <= 0 || d->Nq <= 0 || d->Nk <= 0) return SAGE3_E_SHAPE;
    if (d->D != 64 && d->D != 128) return SAGE3_E_SHAPE;
    if (d->Hq % d->Hkv != 0) return SAGE3_E_SHAPE;
    if (d->dtype != SAGE3_FP16 && d->dtype != SAGE3_BF16) return SAGE3_E_DTYPE;
    // 128-bit loads and stores need every row to start on a 16-byte boundary: strides are multiples of 8 elements
    const int64_t* strides[4] = {d->q_stride, d->k_stride, d->v_stride, d->o_stride};
    for (auto s : strides)
        for (int i = 0; i < 3; ++i)
            if (s[i] < 0 || (s[i] % 8) != 0) return SAGE3_E_STRIDE;
    // index arithmetic inside the kernels is 32-bit for tile counts
    const int64_t nqp = ((int64_t)d->Nq + 127) / 128 * 128, nkp = ((int64_t)d->Nk + 127) / 128 * 128;
    if (nqp > (1 << 24) || nkp > (1 << 24)) return SAGE3_E_TOO_LARGE;
    if ((int64_t)d->B * d->Hq * (nqp / 128) > 0x7fffffffLL) return SAGE3_E_TOO_LARGE;
    // the pre-pass kernels put the (batch, head) index in gridDim.y
    if ((int64_t)d->B * d->Hq > 65535) return SAGE3_E_TOO_LARGE;
    return SAGE3_OK;
}

int layout(const Sage3Desc* d, Sage3Workspace* w) {
    const int rc = validate(d);
    if (rc != SAGE3_OK) return rc;
    if (!w) return SAGE3_E_NULL;
    const size_t B = d->B, Hq = d->Hq, Hkv = d->Hkv, D = d->D;
    const size_t nqp = ((size_t)d->Nq + 127) / 128 * 128, nkp = ((size_t)d->Nk + 127) / 128 * 128;
    const size_t nqm = d->per_block_mean ? nqp / 128 : 1;
    const size_t kch_k = ((size_t)d->Nk + sage3::kRowsPerChunk - 1) / sage3::kRowsPerChunk;
    const size_t kch_q = ((size_t)d->Nq + sage3::kRowsPerChunk - 1) / sage3::kRowsPerChunk;
    size_t part = B * Hkv * kch_k;
    if (!d->per_block_mean && B * Hq * kch_q > part) part = B * Hq * kch_q;
    size_t off = 0;
    w->status = off;  off += align_up(64 * sizeof(int32_t));
    w->kpart = off;   off += align_up(part * D * sizeof(float));
    w->km = off;      off += align_up(B * Hkv * D * 2);
    w->qm = off;      off += align_up(B * Hq * nqm * D * 2);
    w->delta = off;   off += align_up(B * Hq * nqm * nkp * 2);
    w->q_codes = off; off += align_up(B * Hq * nqp * (D / 2));
    w->q_sf = off;    off += align_up(B * Hq * (nqp / 128) * (D / 64) * 512);
    w->k_codes = off; off += align_up(B * Hkv * nkp * (D / 2));
    w->k_sf = off;    off += align_up(B * Hkv * (nkp / 128) * (D / 64) * 512);
    w->v_codes = off; off += align_up(B * Hkv * D * (nkp / 2));
    w->v_sf = off;    off += align_up(B * Hkv * (nkp / 128) * 1024);
    w->qkm = off;     off += align_up(B * Hq * nqp * sizeof(float));
    w->total_bytes = off;
    w->nq_pad = (int32_t)nqp;
    w->nk_pad = (int32_t)nkp;
    w->nqm = (int32_t)nqm;
    w->kchunks = (int32_t)kch_k;
    return SAGE3_OK;
}

int check_arch() {
    int dev = 0, major = 0, minor = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return SAGE3_E_CUDA;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return SAGE3_E_CUDA;
    if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return SAGE3_E_CUDA;
    return (major == 10 && minor == 0) ? SAGE3_OK : SAGE3_E_ARCH;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Status words: [0, 32) belong to the pre-pass, [32, 64) to the attention kernel.  Each stage clears its own half only,
// so a wait the pre-pass gave up on is still there after the attention launch (whose CTAs read it and exit at once).
constexpr int kStatusWords = 64, kAttnStatusWord = 32;

// checks a Sage3Parts argument and converts it; `align`: required alignment of every base pointer
int to_parts(const Sage3Parts* in, int64_t rows_total, sage3::PartsPtr* out) {
    if (!in) return SAGE3_E_NULL;
    if (in->parts < 1 || in->parts > sage3::kMaxParts || in->rows_per_part <= 0) return SAGE3_E_SHAPE;
    if ((int64_t)in->parts * in->rows_per_part < rows_total) return SAGE3_E_SHAPE;
    *out = sage3::PartsPtr{};
    for (int i = 0; i < in->parts; ++i) {
        if (!in->base[i]) return SAGE3_E_NULL;
        if (!aligned(in->base[i], 16)) return SAGE3_E_ALIGN;
        out->base[i] = in->base[i];
    }
    for (int i = in->parts; i < sage3::kMaxParts; ++i) out->base[i] = in->base[in->parts - 1];
    out->rows = in->parts == 1 ? 0 : in->rows_per_part;
    return SAGE3_OK;
}

sage3::PartsPtr one_part(const void* p) {
    sage3::PartsPtr r = {};
    for (int i = 0; i < sage3::kMaxParts; ++i) r.base[i] = const_cast<void*>(p);
    r.rows = 0;
    return r;
}

int attn_impl(const Sage3Desc* desc, void* ws, const sage3::PartsPtr& out, float* lse, float* debug, void* stream,
              const Sage3Carry* carry = nullptr, const int32_t* cu_q = nullptr, const int32_t* cu_k = nullptr) {
    Sage3Workspace w;
    int rc = layout(desc, &w);
    if (rc != SAGE3_OK) return rc;
    if (!ws) return SAGE3_E_NULL;
    if (!out.base[0] && !(carry && carry->o_out)) return SAGE3_E_NULL;      // somewhere the result must go
    if (lse != nullptr && !aligned(lse, 4)) return SAGE3_E_ALIGN;
    if (!aligned(ws, kWsAlign) || !aligned(out.base[0], 16)) return SAGE3_E_ALIGN;
    if (carry) {
        if ((carry->o_in != nullptr) != (carry->m_in != nullptr) || (carry->o_in != nullptr) != (carry->l_in != nullptr)) return SAGE3_E_NULL;
        if ((carry->o_out != nullptr) != (carry->m_out != nullptr) || (carry->o_out != nullptr) != (carry->l_out != nullptr)) return SAGE3_E_NULL;
        if (!aligned(carry->o_in, 16) || !aligned(carry->o_out, 16) || !aligned(carry->m_in, 4) || !aligned(carry->l_in, 4) ||
            !aligned(carry->m_out, 4) || !aligned(carry->l_out, 4))
            return SAGE3_E_ALIGN;
    }
    rc = check_arch();
    if (rc != SAGE3_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* base = static_cast<uint8_t*>(ws);
    if (cudaMemsetAsync(base + w.status + kAttnStatusWord * sizeof(int32_t), 0, (kStatusWords - kAttnStatusWord) * sizeof(int32_t), st) !=
        cudaSuccess)
        return SAGE3_E_CUDA;
    sage3::AttnArgs a;
    a.B = desc->B; a.Hq = desc->Hq; a.Hkv = desc->Hkv; a.Nq = desc->Nq; a.Nk = desc->Nk; a.D = desc->D;
    a.Nq_p = w.nq_pad; a.Nk_p = w.nk_pad; a.nqm = w.nqm;
    a.is_causal = desc->is_causal != 0;
    a.is_bf16 = desc->dtype == SAGE3_BF16;
    a.sm_scale = desc->sm_scale > 0.f ? desc->sm_scale : 1.0f / sqrtf((float)desc->D);
    a.sm_scale_per_head = desc->sm_scale_per_head;
    a.delta = base + w.delta;
    a.q_codes = base + w.q_codes; a.q_sf = base + w.q_sf;
    a.k_codes = base + w.k_codes; a.k_sf = base + w.k_sf;
    a.v_codes = base + w.v_codes; a.v_sf = base + w.v_sf;
    a.out = out;
    a.lse = lse;
    a.qkm = reinterpret_cast<const float*>(base + w.qkm);
    for (int i = 0; i < 3; ++i) a.os[i] = desc->o_stride[i];
    a.carry_o_in = carry ? carry->o_in : nullptr; a.carry_m_in = carry ? carry->m_in : nullptr; a.carry_l_in = carry ? carry->l_in : nullptr;
    a.carry_o_out = carry ? carry->o_out : nullptr; a.carry_m_out = carry ? carry->m_out : nullptr; a.carry_l_out = carry ? carry->l_out : nullptr;
    a.causal_shift = (carry && carry->use_causal_shift) ? carry->causal_shift : desc->Nk - desc->Nq;
    a.status = reinterpret_cast<int*>(base + w.status) + kAttnStatusWord;
    a.prepass_status = reinterpret_cast<const int*>(base + w.status);
    a.cu_q = cu_q; a.cu_k = cu_k;
#ifdef SAGE3_DEV_TRACE
    a.debug = debug;
#else
    (void)debug;
#endif
    int drv = 0;
    return sage3::launch_attn(a, st, &drv) == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

// One warp waits on a barrier that nobody ever arrives on, with a limit of about a millisecond: exercises the
// bounded-wait path (status word, abort flag, normal kernel exit) without hanging anything.
__global__ void wait_timeout_selftest_kernel(int* status) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        sage3::mbar_init(sage3::smem_u32(&bar), 1);
        sage3::mbar_fence_init();
    }
    __syncthreads();
    sage3::mbar_wait(sage3::smem_u32(&bar), 0, &abort_flag, status, sage3::kWaitSelfTest, 2000000LL);
}

// Slab copy: blockIdx.y = slab, blockIdx.x = piece of the slab; 8 independent 16-byte loads per thread in flight.
struct SlabCopyArgs {
    int n1, n2;
    long long ds0, ds1, ds2, ss0, ss1, ss2;   // in 16-byte units
    long long slab_v;                          // 16-byte vectors per slab
};
__global__ void __launch_bounds__(256) slab_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, SlabCopyArgs a) {
    const int slab = blockIdx.y;
    const int i2 = slab % a.n2, i1 = (slab / a.n2) % a.n1, i0 = slab / (a.n2 * a.n1);
    const uint4* s = src + i0 * a.ss0 + i1 * a.ss1 + i2 * a.ss2;
    uint4* d = dst + i0 * a.ds0 + i1 * a.ds1 + i2 * a.ds2;
    const long long base = (long long)blockIdx.x * (256 * 8) + threadIdx.x;
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long idx = base + i * 256;
        if (idx < a.slab_v) v[i] = __ldg(s + idx);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long idx = base + i * 256;
        if (idx < a.slab_v) d[idx] = v[i];
    }
}

// Merge of a partial attention result into the running one: 8 channels per thread.
template <typename T>
__global__ void __launch_bounds__(256) merge_partial_kernel(float* __restrict__ acc, float* __restrict__ lse_acc,
                                                            const T* __restrict__ o_part, const float* __restrict__ lse_part,
                                                            T* __restrict__ out, long long rows, int D, int first) {
    const int tpr = D / 8;                                   // threads per row
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    const long long r = idx / tpr;
    const int c = (int)(idx % tpr) * 8;
    if (r >= rows) return;
    const float lp = lse_part[r];
    const float la = first ? -INFINITY : lse_acc[r];
    const float mx = fmaxf(la, lp);
    float ln = mx, wa = 0.f, wp = 0.f;
    if (mx != -INFINITY) {
        const float ea = __expf(la - mx), ep = __expf(lp - mx);
        ln = mx + __logf(ea + ep);
        wa = __expf(la - ln);
        wp = __expf(lp - ln);
    }
    const uint4 raw = *reinterpret_cast<const uint4*>(o_part + r * D + c);
    const T* ov = reinterpret_cast<const T*>(&raw);
    float a[8];
    if (first) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = 0.f;
    } else {
        const float4 a0 = *reinterpret_cast<const float4*>(acc + r * D + c), a1 = *reinterpret_cast<const float4*>(acc + r * D + c + 4);
        a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = a[i] * wa + static_cast<float>(ov[i]) * wp;
    *reinterpret_cast<float4*>(acc + r * D + c) = make_float4(a[0], a[1], a[2], a[3]);
    *reinterpret_cast<float4*>(acc + r * D + c + 4) = make_float4(a[4], a[5], a[6], a[7]);
    if (out != nullptr) {
        uint4 w;
        T* wv = reinterpret_cast<T*>(&w);
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[i] = static_cast<T>(a[i]);
        *reinterpret_cast<uint4*>(out + r * D + c) = w;
    }
    __syncwarp();
    if (c == 0) lse_acc[r] = ln;       // (every thread of the row has read lse_acc above: rows never straddle warps, D/8 divides 32)
}

}  // namespace

extern "C" {

SAGE3_API int sage3_version(void) { return SAGE3_ABI_VERSION; }

SAGE3_API const char* sage3_strerror(int code) {
    switch (code) {
        case SAGE3_OK: return "ok";
        case SAGE3_E_NULL: return "a required pointer is NULL";
        case SAGE3_E_SHAPE: return "unsupported shape (D must be 64 or 128, Hq a multiple of Hkv, sizes positive)";
        case SAGE3_E_DTYPE: return "dtype must be SAGE3_FP16 or SAGE3_BF16";
        case SAGE3_E_STRIDE: return "strides must be non-negative multiples of 8 elements with the last dimension contiguous";
        case SAGE3_E_ALIGN: return "pointer alignment: tensors 16 bytes, workspace 256 bytes";
        case SAGE3_E_ARCH: return "the current CUDA device is not compute capability 10.0 (B200)";
        case SAGE3_E_CUDA: return "a CUDA call or kernel launch failed";
        case SAGE3_E_TOO_LARGE: return "a size exceeds a fixed limit of this entry point";
        case SAGE3_E_DEVICE_WAIT: return "a bounded device-side wait gave up (see the status word)";
        default: return "unknown status code";
    }
}

SAGE3_API int sage3_workspace_layout(const Sage3Desc* desc, Sage3Workspace* ws) { return layout(desc, ws); }

SAGE3_API size_t sage3_workspace_bytes(const Sage3Desc* desc) {
    Sage3Workspace w;
    return layout(desc, &w) == SAGE3_OK ? w.total_bytes : 0;
}

static int prepass_impl(const Sage3Desc* desc, const sage3::PartsPtr& q, const sage3::PartsPtr& k, const sage3::PartsPtr& v,
                        const void* km_in, void* ws, void* stream, const int32_t* cu_q = nullptr, const int32_t* cu_k = nullptr) {
    Sage3Workspace w;
    int rc = layout(desc, &w);
    if (rc != SAGE3_OK) return rc;
    if (!ws) return SAGE3_E_NULL;
    if (!aligned(ws, kWsAlign)) return SAGE3_E_ALIGN;
    rc = check_arch();
    if (rc != SAGE3_OK) return rc;
    uint8_t* base = static_cast<uint8_t*>(ws);
    sage3::PrepassArgs a;
    a.q = q; a.k = k; a.v = v;
    for (int i = 0; i < 3; ++i) {
        a.qs[i] = desc->q_stride[i];
        a.ks[i] = desc->k_stride[i];
        a.vs[i] = desc->v_stride[i];
    }
    a.B = desc->B; a.Hq = desc->Hq; a.Hkv = desc->Hkv; a.Nq = desc->Nq; a.Nk = desc->Nk; a.D = desc->D;
    a.Nq_p = w.nq_pad; a.Nk_p = w.nk_pad; a.nqm = w.nqm;
    a.per_block_mean = desc->per_block_mean != 0;
    a.is_bf16 = desc->dtype == SAGE3_BF16;
    a.kchunks_k = w.kchunks;
    a.kchunks_q = (desc->Nq + sage3::kRowsPerChunk - 1) / sage3::kRowsPerChunk;
    a.kpart = reinterpret_cast<float*>(base + w.kpart);
    a.km = base + w.km; a.qm = base + w.qm; a.delta = base + w.delta;
    a.q_codes = base + w.q_codes; a.q_sf = base + w.q_sf;
    a.k_codes = base + w.k_codes; a.k_sf = base + w.k_sf;
    a.v_codes = base + w.v_codes; a.v_sf = base + w.v_sf;
    a.qkm = reinterpret_cast<float*>(base + w.qkm);
    a.status = reinterpret_cast<int*>(base + w.status);
    a.cu_q = cu_q; a.cu_k = cu_k;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(base + w.status, 0, kStatusWords * sizeof(int32_t), st) != cudaSuccess) return SAGE3_E_CUDA;
    a.km_given = km_in != nullptr;
    if (km_in != nullptr &&
        cudaMemcpyAsync(a.km, km_in, (size_t)desc->B * desc->Hkv * desc->D * 2, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return SAGE3_E_CUDA;
    return sage3::launch_prepass(a, st) == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

SAGE3_API int sage3_prepass(const Sage3Desc* desc, const void* q, const void* k, const void* v, void* ws, void* stream) {
    if (!q || !k || !v) return SAGE3_E_NULL;
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16)) return SAGE3_E_ALIGN;
    return prepass_impl(desc, one_part(q), one_part(k), one_part(v), nullptr, ws, stream);
}

// Packed variable-length batch: desc->B sequences, desc->Nq / desc->Nk the longest of them, sequence b owning rows
// cu[b] .. cu[b + 1] of the packed tensors.  One launch of every kernel covers the whole batch; the workspace has the
// layout of a uniform batch of the maximum lengths, and CTAs beyond a sequence's own length leave at once.
SAGE3_API int sage3_fwd_varlen(const Sage3Desc* desc, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const void* q,
                               const void* k, const void* v, void* out, float* lse, void* ws, void* stream) {
    if (!desc || !cu_seqlens_q || !cu_seqlens_k || !q || !k || !v || !out) return SAGE3_E_NULL;
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(cu_seqlens_q, 4) || !aligned(cu_seqlens_k, 4)) return SAGE3_E_ALIGN;
    const int rc = prepass_impl(desc, one_part(q), one_part(k), one_part(v), nullptr, ws, stream, cu_seqlens_q, cu_seqlens_k);
    if (rc != SAGE3_OK) return rc;
    return attn_impl(desc, ws, one_part(out), lse, nullptr, stream, nullptr, cu_seqlens_q, cu_seqlens_k);
}

SAGE3_API int sage3_prepass_kmean(const Sage3Desc* desc, const void* q, const void* k, const void* v, const void* km, void* ws,
                                  void* stream) {
    if (!q || !k || !v || !km) return SAGE3_E_NULL;
    if (!aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(km, 2)) return SAGE3_E_ALIGN;
    return prepass_impl(desc, one_part(q), one_part(k), one_part(v), km, ws, stream);
}

SAGE3_API int sage3_prepass_parts(const Sage3Desc* desc, const Sage3Parts* q, const Sage3Parts* k, const Sage3Parts* v, void* ws,
                                  void* stream) {
    if (!desc) return SAGE3_E_NULL;
    sage3::PartsPtr qp, kp, vp;
    int rc = to_parts(q, desc->Nq, &qp);
    if (rc == SAGE3_OK) rc = to_parts(k, desc->Nk, &kp);
    if (rc == SAGE3_OK) rc = to_parts(v, desc->Nk, &vp);
    if (rc != SAGE3_OK) return rc;
    return prepass_impl(desc, qp, kp, vp, nullptr, ws, stream);
}

SAGE3_API int sage3_attn_fwd_carry(const Sage3Desc* desc, void* ws, const Sage3Carry* carry, void* out, float* lse, void* stream) {
    if (!carry) return SAGE3_E_NULL;
    return attn_impl(desc, ws, one_part(out), lse, nullptr, stream, carry);
}

SAGE3_API int sage3_attn_fwd_parts(const Sage3Desc* desc, void* ws, const Sage3Parts* out, float* lse, void* stream) {
    if (!desc) return SAGE3_E_NULL;
    sage3::PartsPtr op;
    const int rc = to_parts(out, desc->Nq, &op);
    if (rc != SAGE3_OK) return rc;
    return attn_impl(desc, ws, op, lse, nullptr, stream);
}

// ---- memory that other processes of the node can map (for the peer-to-peer form of sequence parallelism) ----------
SAGE3_API int sage3_shared_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
    if (!ptr || !handle || bytes == 0) return SAGE3_E_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (cudaMalloc(ptr, bytes) != cudaSuccess) return SAGE3_E_CUDA;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) {
        cudaFree(*ptr);
        *ptr = nullptr;
        return SAGE3_E_CUDA;
    }
    memcpy(handle, &h, 64);
    return SAGE3_OK;
}

SAGE3_API int sage3_shared_open(const unsigned char handle[64], void** ptr) {
    if (!ptr || !handle) return SAGE3_E_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

SAGE3_API int sage3_shared_close(void* ptr) {
    if (!ptr) return SAGE3_E_NULL;
    return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

SAGE3_API int sage3_shared_free(void* ptr) {
    if (!ptr) return SAGE3_E_NULL;
    return cudaFree(ptr) == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

SAGE3_API int sage3_attn_fwd(const Sage3Desc* desc, void* ws, void* out, float* lse, void* stream) {
    return attn_impl(desc, ws, one_part(out), lse, nullptr, stream);
}

#ifdef SAGE3_DEV_TRACE
// development builds only (not declared in the public header): attention with the instrumentation dump
SAGE3_API int sage3_attn_fwd_debug(const Sage3Desc* desc, void* ws, void* out, float* debug, void* stream) {
    return attn_impl(desc, ws, one_part(out), nullptr, debug, stream);
}
#endif

SAGE3_API int sage3_fwd(const Sage3Desc* desc, const void* q, const void* k, const void* v, void* ws, void* out, float* lse,
              void* stream) {
    const int rc = sage3_prepass(desc, q, k, v, ws, stream);
    if (rc != SAGE3_OK) return rc;
    return sage3_attn_fwd(desc, ws, out, lse, stream);
}

SAGE3_API int sage3_selftest_wait_timeout(void* ws, void* stream) {
    if (!ws) return SAGE3_E_NULL;
    const int rc = check_arch();
    if (rc != SAGE3_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemsetAsync(ws, 0, 64 * sizeof(int32_t), st) != cudaSuccess) return SAGE3_E_CUDA;
    wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(static_cast<int*>(ws));
    return cudaGetLastError() == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

SAGE3_API int sage3_slab_copy(void* dst, const void* src, int32_t n0, int32_t n1, int32_t n2, const int64_t ds[3],
                              const int64_t ss[3], int64_t slab_bytes, void* stream) {
    if (!dst || !src || !ds || !ss) return SAGE3_E_NULL;
    if (n0 <= 0 || n1 <= 0 || n2 <= 0 || slab_bytes <= 0) return SAGE3_E_SHAPE;
    if ((int64_t)n0 * n1 * n2 > 65535) return SAGE3_E_TOO_LARGE;
    if (!aligned(dst, 16) || !aligned(src, 16) || slab_bytes % 16) return SAGE3_E_ALIGN;
    for (int i = 0; i < 3; ++i)
        if (ds[i] % 16 || ss[i] % 16) return SAGE3_E_STRIDE;
    SlabCopyArgs a;
    a.n1 = n1; a.n2 = n2;
    a.ds0 = ds[0] / 16; a.ds1 = ds[1] / 16; a.ds2 = ds[2] / 16;
    a.ss0 = ss[0] / 16; a.ss1 = ss[1] / 16; a.ss2 = ss[2] / 16;
    a.slab_v = slab_bytes / 16;
    const long long pieces = (a.slab_v + 256 * 8 - 1) / (256 * 8);
    if (pieces > 0x7fffffffLL) return SAGE3_E_TOO_LARGE;
    slab_copy_kernel<<<dim3((unsigned)pieces, (unsigned)(n0 * n1 * n2)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(dst), static_cast<const uint4*>(src), a);
    return cudaGetLastError() == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

SAGE3_API int sage3_merge_partial(float* acc, float* lse_acc, const void* o_part, const float* lse_part, void* out,
                                  int64_t rows, int32_t D, int32_t dtype, int32_t first, void* stream) {
    if (!acc || !lse_acc || !o_part || !lse_part) return SAGE3_E_NULL;
    if (rows <= 0 || D <= 0 || D % 8 != 0 || (256 % (D / 8)) != 0 || (32 % (D / 8)) != 0) return SAGE3_E_SHAPE;
    if (dtype != SAGE3_FP16 && dtype != SAGE3_BF16) return SAGE3_E_DTYPE;
    if (!aligned(acc, 16) || !aligned(o_part, 16) || (out && !aligned(out, 16))) return SAGE3_E_ALIGN;
    const long long threads = (long long)rows * (D / 8);
    const long long blocks = (threads + 255) / 256;
    if (blocks > 0x7fffffffLL) return SAGE3_E_TOO_LARGE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == SAGE3_BF16)
        merge_partial_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(acc, lse_acc, static_cast<const __nv_bfloat16*>(o_part),
                                                                             lse_part, static_cast<__nv_bfloat16*>(out), rows, D, first);
    else
        merge_partial_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(acc, lse_acc, static_cast<const __half*>(o_part), lse_part,
                                                                     static_cast<__half*>(out), rows, D, first);
    return cudaGetLastError() == cudaSuccess ? SAGE3_OK : SAGE3_E_CUDA;
}

SAGE3_API int sage3_check_status(const void* ws, int32_t* word, void* stream) {
    if (!ws) return SAGE3_E_NULL;
    int32_t host[64];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(host, ws, sizeof(host), cudaMemcpyDeviceToHost, st) != cudaSuccess) return SAGE3_E_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return SAGE3_E_CUDA;
    for (int i = 0; i < 64; ++i)
        if (host[i] != 0) {
            if (word) *word = host[i];
            return SAGE3_E_DEVICE_WAIT;
        }
    if (word) *word = 0;
    return SAGE3_OK;
}

}  // extern "C"
