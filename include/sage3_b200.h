/*
 * sage3_b200.h -- C ABI of libsage3_b200.so: SageAttention3 (NVFP4 attention) for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; no framework types cross this boundary.  Every buffer, including the
 * workspace, is allocated by the caller and must be device memory of the current CUDA device.  All
 * work is enqueued on the caller's stream; the functions return as soon as the launches are queued.
 * Functions return 0 on success and a negative SAGE3_E_* code otherwise (see sage3_strerror); they
 * never throw and never terminate the process.
 *
 * The entry points replace the two pybind11 modules of the reference
 * (paths inside the reference project, sageattention3_blackwell/sageattn3/...):
 *   fp4quant_cuda.scaled_fp4_quant / _permute / _trans   quantization/fp4_quantization_4d.cu:388-628
 *   fp4attn_cuda.fwd                                     blackwell/api.cu:203-341
 * and the Python pre-processing in front of them (api.py:75-92, preprocess_qkv).
 */
#ifndef SAGE3_B200_H_
#define SAGE3_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAGE3_ABI_VERSION 4

#if defined(__GNUC__)
#define SAGE3_API __attribute__((visibility("default")))
#else
#define SAGE3_API
#endif

enum {
    SAGE3_OK = 0,
    SAGE3_E_NULL = -1,        /* a required pointer is NULL */
    SAGE3_E_SHAPE = -2,       /* unsupported shape: D not in {64,128}, Hq % Hkv != 0, sizes <= 0 ... */
    SAGE3_E_DTYPE = -3,       /* dtype is neither SAGE3_FP16 nor SAGE3_BF16 */
    SAGE3_E_STRIDE = -4,      /* a stride breaks the 16-byte alignment the vector loads need */
    SAGE3_E_ALIGN = -5,       /* a base pointer is not 16-byte (workspace: 256-byte) aligned */
    SAGE3_E_ARCH = -6,        /* the current device is not compute capability 10.0 */
    SAGE3_E_CUDA = -7,        /* a CUDA runtime / driver call or a kernel launch failed */
    SAGE3_E_TOO_LARGE = -8,   /* a size exceeds a fixed limit of the entry point */
    SAGE3_E_DEVICE_WAIT = -9  /* (sage3_check_status) a bounded device-side wait gave up */
};

enum { SAGE3_FP16 = 0, SAGE3_BF16 = 1 };

/*
 * Problem description.  Tensors are addressed as x[b][h][n][d] with the element strides given here and
 * d contiguous, so "HND" ([B,H,N,D]) and "NHD" ([B,N,H,D]) callers use the same code path
 * (the keyword surface of sageattention/core.py:79-157 `tensor_layout`).
 * GQA: query head h reads kv head h / (Hq / Hkv).  Causal masks are bottom-right aligned on the REAL lengths
 * (key j is visible to query i iff j <= i + Nk - Nq; the flash-attention convention).  The reference aligns on the
 * lengths padded to 128 (blackwell/mainloop_tma_ws.h:286-289 works on the padded sizes): identical when Nq and Nk are
 * multiples of 128, deliberately different otherwise (e.g. Nq = 300, Nk = 500: a shift of 200 here, 128 there).
 */
typedef struct Sage3Desc {
    int32_t B, Hq, Hkv, Nq, Nk, D;
    int32_t dtype;            /* SAGE3_FP16 | SAGE3_BF16: element type of q, k, v and out */
    int32_t is_causal;
    int32_t per_block_mean;   /* 1: Q smoothed per 128-row block (api.py:86-87); 0: one mean per head (api.py:88-90) */
    int32_t reserved;
    int64_t q_stride[3];      /* element strides of q for (b, h, n) */
    int64_t k_stride[3];
    int64_t v_stride[3];
    int64_t o_stride[3];
    float sm_scale;           /* softmax scale; <= 0 selects D^-0.5 (api.py:127) */
    int32_t reserved2;
    const float* sm_scale_per_head;   /* optional device array [Hq] overriding sm_scale; NULL if unused */
} Sage3Desc;

/*
 * Byte offsets of the regions inside the workspace (all multiples of 1024).  Np = N rounded up to 128.
 *   status   int32[64]                        device-written status words (0 = fine): [0, 32) pre-pass, [32, 64) attention;
 *                                             each stage clears its own half, so sage3_check_status after sage3_fwd sees both
 *   kpart    fp32 [B*Hkv][chunks][D]          scratch: partial column sums of K (and of Q when per_block_mean = 0)
 *   km       dtype[B][Hkv][D]                 mean of K over its Nk tokens
 *   qm       dtype[B][Hq][nqm][D]             Q means; nqm = Nq_p/128, or 1 when per_block_mean = 0
 *   delta    dtype[B][Hq][nqm][Nk_p]          qm . k'^T  (api.py:91)
 *   q_codes  u8   [B][Hq][Nq_p][D/2]          E2M1, element 2i in bits 0-3 of byte i
 *   q_sf     u8   [B][Hq][Nq_p/128][D/64][512]   E4M3 scales in 128-row x 4-scale atoms:
 *                                              byte (r % 32) * 16 + (r / 32) * 4 + (c % 4), atom index c / 4
 *   k_codes, k_sf                             same for K (kv heads), natural token order
 *   v_codes  u8   [B][Hkv][D][Nk_p/2]         V transposed, microblocks of 16 consecutive tokens
 *   v_sf     u8   [B][Hkv][Nk_p/128][2][512]  atoms with r = channel, c = (token % 128) / 16
 *   qkm      fp32 [B][Hq][Nq_p]               q . km per query row (the part of q k^T that K smoothing removes;
 *                                             core.py:289-293 `lse_correction`), used by the LSE output
 */
typedef struct Sage3Workspace {
    size_t status, kpart, km, qm, delta, q_codes, q_sf, k_codes, k_sf, v_codes, v_sf, qkm;
    size_t total_bytes;
    int32_t nq_pad, nk_pad, nqm, kchunks;
} Sage3Workspace;

/* ABI version of the loaded library (SAGE3_ABI_VERSION at build time). */
SAGE3_API int sage3_version(void);

/* Static, never-NULL text for a status code. */
SAGE3_API const char* sage3_strerror(int code);

/* Validates `desc` and fills `ws` with the workspace layout.  No device work.
 * Replaces the shape arithmetic of api.py:94-116 and the checks of blackwell/api.cu:219-286. */
SAGE3_API int sage3_workspace_layout(const Sage3Desc* desc, Sage3Workspace* ws);

/* Bytes of workspace `desc` needs (0 if desc is invalid). */
SAGE3_API size_t sage3_workspace_bytes(const Sage3Desc* desc);

/*
 * Pre-pass: K smoothing, Q smoothing, delta_s, and NVFP4 quantization of Q, K and V-transposed into
 * `ws`.  Never writes to q, k or v (the reference smooths K in place, api.py:84).
 * Replaces preprocess_qkv (api.py:75-92) + scale_and_quant_fp4 / _permute / _transpose (api.py:94-116)
 * and the kernels behind them (fp4_quantization_4d.cu:133-386).
 * `stream` is a cudaStream_t.
 */
SAGE3_API int sage3_prepass(const Sage3Desc* desc, const void* q, const void* k, const void* v, void* ws, void* stream);

/*
 * Attention over a workspace filled by sage3_prepass with the same `desc`: out[b][h][n][d] in `dtype`
 * with the strides of desc->o_stride.  Replaces fp4attn_cuda.fwd (blackwell/api.cu:203-341) and the
 * final slice of api.py:151 (rows beyond Nq are never written).
 * `lse`: NULL, or a device array fp32 [B][Hq][Nq] that receives the natural-log log-sum-exp of the scaled scores
 * of every query row, ln sum_k exp(sm_scale * q.k), computed from the quantized scores plus sm_scale * q.km as
 * sageattention/core.py:327 does for its kernels (-inf for a row without visible keys).
 */
SAGE3_API int sage3_attn_fwd(const Sage3Desc* desc, void* ws, void* out, float* lse, void* stream);

/*
 * Packed variable-length batch in one launch of every kernel (replaces the reference's sageattn_varlen entry,
 * sageattention/core.py:334-448, which takes the same cu_seqlens / max_seqlen arguments).  q is [total_q][Hq][D], k and
 * v are [total_k][Hkv][D], out is [total_q][Hq][D]; sequence b owns query rows cu_seqlens_q[b] .. cu_seqlens_q[b + 1]
 * and key rows cu_seqlens_k[b] .. cu_seqlens_k[b + 1] (device arrays of desc->B + 1 int32, never read by the host).
 * In `desc`: B = number of sequences, Nq / Nk = the longest query / key length (lengths beyond them are clamped),
 * stride[1] = head stride, stride[2] = token stride, stride[0] unused.  Every sequence is smoothed, quantized and
 * attended exactly as a sage3_fwd call on it alone would be (its own K mean, its own padding to 128 rows, causal mask
 * aligned on its own lengths); a sequence without keys gets zeros.  The workspace is the one of a uniform batch of B
 * entries of the maximum lengths (sage3_workspace_bytes(desc)).  `lse`: NULL, or fp32 [B][Hq][desc->Nq] that receives the
 * log-sum-exp of every query row of sequence b at [b][h][0 .. len_q(b)) (entries beyond a sequence's length are not
 * written).  No per-call K mean, no carried state.
 */
SAGE3_API int sage3_fwd_varlen(const Sage3Desc* desc, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const void* q,
                               const void* k, const void* v, void* out, float* lse, void* ws, void* stream);

/*
 * Column means from partial column sums: mean_out[r][d] (dtype, [rows][D]) = the sum over c = 0 .. chunks - 1, in that
 * order, of part[r][c][d] (fp32, [rows][chunks][D]), times 1 / count, rounded once -- the second half of the K-mean stage
 * (api.py:84) on its own.  Context-parallel callers gather the 512-row partial sums that sage3_prepass leaves in the
 * `kpart` region of every rank's workspace, shard after shard, and obtain the K mean of the whole sequence exactly as a
 * single call forms it (then passed to sage3_prepass_kmean).
 */
SAGE3_API int sage3_mean_from_partial_sums(const float* part, int32_t rows, int32_t chunks, int32_t D, int32_t dtype, int64_t count,
                                           void* mean_out, void* stream);

/*
 * sage3_prepass with the K mean supplied by the caller: `km` is a device array dtype[B][Hkv][D] that is used instead of
 * the mean over this call's Nk tokens.  For context-parallel callers whose K is one shard of a longer sequence: they
 * pass the mean over all shards, so every shard is smoothed exactly as the whole sequence would be (api.py:84 takes
 * the mean over the whole sequence).
 */
SAGE3_API int sage3_prepass_kmean(const Sage3Desc* desc, const void* q, const void* k, const void* v, const void* km, void* ws,
                                  void* stream);

/*
 * Attention over one key range of a longer attention, with the accumulator state carried from call to call.
 * One attention over keys [0, Nk_total) may be computed as several calls over consecutive key ranges, walked from the
 * LAST range to the FIRST (the order in which the kernel walks the key blocks of a single call, mainloop_tma_ws.h:509,
 * 865): every call but the first passes the state the previous one left (o_in / m_in / l_in), every call but the last
 * asks for it (o_out / m_out / l_out; `out` may then be NULL), the last call writes `out` (and `lse`).  When every
 * range but the last is a multiple of 128 keys and the pre-pass of every range used the K mean of the whole sequence
 * (sage3_prepass_kmean), the result equals the single call's bit for bit: the same blocks in the same order with the
 * same arithmetic.  This is the building block of context-parallel ("ring") attention and of key/value streaming; the
 * reference offers `return_lse` for that use (sageattention/core.py:120-122), which cannot reproduce the single call
 * because the FP4 rounding of P depends on the running maximum when a block is processed.
 *   o: fp32 [B][Hq][Nq][D] unnormalized accumulator; m: fp32 [B][Hq][Nq] running maximum of the smoothed scores; l: fp32
 *   [B][Hq][Nq][2] the two partial row sums the kernel keeps per row (keys 0-63 and 64-127 of every block; carried
 *   separately so that the additions stay in the single call's order).  In-place (o_in == o_out ...) is allowed.  With is_causal, `causal_shift` (when use_causal_shift != 0)
 *   replaces Nk - Nq in the mask  key j visible to query i  <=>  j <= i + causal_shift,  j counted inside this call's
 *   key range: pass  Nk_total - Nq - first_key_of_the_range.
 */
typedef struct Sage3Carry {
    const float* o_in;
    const float* m_in;
    const float* l_in;
    float* o_out;
    float* m_out;
    float* l_out;
    int32_t use_causal_shift;
    int32_t causal_shift;
} Sage3Carry;
SAGE3_API int sage3_attn_fwd_carry(const Sage3Desc* desc, void* ws, const Sage3Carry* carry, void* out, float* lse, void* stream);

/*
 * A tensor whose token dimension is split into `parts` equal pieces that live in different buffers: piece p holds tokens
 * [p * rows_per_part, (p + 1) * rows_per_part) and is addressed with the (b, h, n) strides of Sage3Desc, n counted from
 * the start of the piece.  The buffers may be memory of other GPUs of the node mapped into this process (see
 * sage3_shared_open): the kernels touch them with plain loads and stores only.  This is the peer-to-peer form of the
 * sequence-parallel exchange that the reference leaves to xfuser (example/parallel_sageattn_cogvideo.py:8-14, 89-95):
 * every rank's token shard stays where it is, the pre-pass of the rank that owns a head reads it from there, and the
 * attention epilogue writes each output row into the shard of the rank that owns the token.
 */
#define SAGE3_MAX_PARTS 8
typedef struct Sage3Parts {
    int32_t parts;                  /* 1 .. SAGE3_MAX_PARTS */
    int32_t rows_per_part;          /* tokens per piece; parts * rows_per_part >= the tensor's token count */
    void* base[SAGE3_MAX_PARTS];    /* 16-byte aligned; base[p] already points at this call's first (batch, head) */
} Sage3Parts;

/* sage3_prepass / sage3_attn_fwd on token-split tensors.  No counterpart in the reference. */
SAGE3_API int sage3_prepass_parts(const Sage3Desc* desc, const Sage3Parts* q, const Sage3Parts* k, const Sage3Parts* v, void* ws,
                                  void* stream);
SAGE3_API int sage3_attn_fwd_parts(const Sage3Desc* desc, void* ws, const Sage3Parts* out, float* lse, void* stream);

/*
 * Device memory that other processes on the same node can map (CUDA IPC), for the buffers behind Sage3Parts.
 * sage3_shared_alloc: cudaMalloc on the current device + a 64-byte handle to pass to the other processes;
 * sage3_shared_open: maps such a handle into this process (peer access is enabled on first use);
 * sage3_shared_close / sage3_shared_free undo them.  The only entry points of this library that allocate.
 * No counterpart in the reference.
 */
SAGE3_API int sage3_shared_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
SAGE3_API int sage3_shared_open(const unsigned char handle[64], void** ptr);
SAGE3_API int sage3_shared_close(void* ptr);
SAGE3_API int sage3_shared_free(void* ptr);

/* sage3_prepass followed by sage3_attn_fwd on the same stream. */
SAGE3_API int sage3_fwd(const Sage3Desc* desc, const void* q, const void* k, const void* v, void* ws, void* out,
              float* lse, void* stream);

/*
 * Synchronizes `stream`, reads the status words of `ws` back and returns SAGE3_OK or
 * SAGE3_E_DEVICE_WAIT; the first non-zero word is stored in *word when word != NULL.
 * Debugging aid: device-side waits are bounded and report here instead of hanging.
 */
SAGE3_API int sage3_check_status(const void* ws, int32_t* word, void* stream);

/*
 * Failure-reporting self test: launches one warp that waits, with a limit of about a millisecond, on a barrier
 * nobody arrives on.  The kernel returns normally; afterwards sage3_check_status(ws, &word, stream) must report
 * SAGE3_E_DEVICE_WAIT with word == 199.  `ws` needs 256 bytes.  No counterpart in the reference (its only failure
 * handling is `assert` and `exit`, quantization/cuda_utils.h:19-27).
 */
SAGE3_API int sage3_selftest_wait_timeout(void* ws, void* stream);

/*
 * Strided copy of n0 x n1 x n2 contiguous slabs of `slab_bytes` bytes each: slab (i0, i1, i2) goes from
 * src + i0*ss[0] + i1*ss[1] + i2*ss[2] to dst + i0*ds[0] + i1*ds[1] + i2*ds[2] (strides in bytes).  Everything
 * (pointers, strides, slab_bytes) must be a multiple of 16.  This is the head <-> token regrouping around the two
 * all-to-alls of sequence-parallel attention (a slab = the [tokens, D] block of one (batch, head)).  No counterpart in
 * the reference, whose parallel example leaves the exchange to xfuser (example/parallel_sageattn_cogvideo.py:8-14).
 */
SAGE3_API int sage3_slab_copy(void* dst, const void* src, int32_t n0, int32_t n1, int32_t n2, const int64_t ds[3],
                              const int64_t ss[3], int64_t slab_bytes, void* stream);

/*
 * Merges one partial attention result into a running one (context-parallel / ring composition of attention over
 * disjoint key sets, the use `return_lse` exists for: sageattention/core.py:120-122).  For every row r of `rows`:
 *   lse' = log(exp(lse_acc[r]) + exp(lse_part[r]));  acc[r][:] = acc[r][:] * exp(lse_acc[r] - lse') +
 *   o_part[r][:] * exp(lse_part[r] - lse');  lse_acc[r] = lse'.
 * `acc` fp32 [rows][D] and `lse_acc` fp32 [rows] are read and written (ignored on input when first != 0);
 * `o_part` is `dtype` [rows][D] contiguous, `lse_part` fp32 [rows]; when `out` is not NULL the merged rows are also
 * written to it in `dtype` ([rows][D] contiguous).  D must be a multiple of 8.  No counterpart in the reference.
 */
SAGE3_API int sage3_merge_partial(float* acc, float* lse_acc, const void* o_part, const float* lse_part, void* out,
                                  int64_t rows, int32_t D, int32_t dtype, int32_t first, void* stream);

/*
 * Mean of K over its Nk tokens, per (batch, kv-head) and channel -- the first stage of the pre-pass -- for
 * callers that must not allocate device memory and cannot hand over a workspace: for instance a serving
 * engine that gave all device memory to its own pool at start-up, or a latency-critical loop in which a
 * cudaMalloc (and the device-wide synchronization it implies) is not acceptable.  It has no counterpart in
 * the reference.
 *
 * km_out[b][h][d] (element type desc->dtype, B*Hkv*D elements, caller-allocated device memory) receives exactly
 * the values sage3_prepass leaves in the `km` region of its workspace.  Only B, Hkv, Nk, D, dtype and k_stride
 * of `desc` are read.  The partial sums go to a fixed array that lives inside the library image on every GPU
 * that loads it (SAGE3_KMEAN_NOALLOC_MAX_FLOATS floats = 4 MiB, held until the process exits); the call
 * returns SAGE3_E_TOO_LARGE when B*Hkv*ceil(Nk/512)*D exceeds that many floats.  The function calls no
 * cudaMalloc / cudaFree and no allocating library routine.
 *
 * The first call on each device looks the array's device address up (that device must be current); make that
 * first call before any stream capture begins.  All calls on a device share the one array, which keeps the
 * previous call's contents (nothing in it needs clearing: each call overwrites what it reads): two calls
 * whose kernels may overlap on the GPU -- different streams without an ordering between them -- race on it.
 */
#define SAGE3_KMEAN_NOALLOC_MAX_FLOATS (1u << 20)
SAGE3_API int sage3_kmean_noalloc(const Sage3Desc* desc, const void* k, void* km_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SAGE3_B200_H_ */
