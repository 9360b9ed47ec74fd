// Host-visible launch interface between the C ABI (sage3_abi.cu) and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace sage3 {

constexpr int kRowsPerChunk = 512;   // rows per partial column sum (fixes the summation order)
constexpr int kMaxParts = 8;         // a tensor's tokens may be split over this many buffers (one per GPU of a node)

// A tensor whose token dimension is split into equal parts living in different buffers (e.g. the token shards of the
// ranks of a sequence-parallel group, mapped into this process): part p holds tokens [p * rows, (p + 1) * rows).
// rows == 0: one buffer, base[0].
struct PartsPtr {
    void* base[kMaxParts];
    int rows;
};

struct PrepassArgs {
    PartsPtr q, k, v;
    int64_t qs[3], ks[3], vs[3];   // element strides for (b, h, n)
    int B, Hq, Hkv, Nq, Nk, D, Nq_p, Nk_p, nqm;
    int per_block_mean, is_bf16;
    int km_given;                  // the K mean is already in `km` (computed elsewhere): skip its two kernels
    int kchunks_k, kchunks_q;
    float* kpart;
    void *km, *qm, *delta;
    uint8_t *q_codes, *q_sf, *k_codes, *k_sf, *v_codes, *v_sf;
    float* qkm;                    // fp32 [B][Hq][Nq_p]: q . km per query row
    int* status;                   // device status words (bounded waits report here)
    // packed variable-length sequences (both nullptr: every batch entry has Nq / Nk tokens): device int32 [B + 1], entry b
    // owns rows cu[b] .. cu[b + 1] of the packed tensor; Nq / Nk are then the maximum lengths, stride 0 is unused
    const int *cu_q, *cu_k;
};

struct AttnArgs {
    int B, Hq, Hkv, Nq, Nk, D, Nq_p, Nk_p, nqm;
    int is_causal, is_bf16;
    float sm_scale;                 // already resolved (> 0)
    const float* sm_scale_per_head; // device [Hq] or nullptr
    const void* delta;              // dtype [B][Hq][nqm][Nk_p]
    const uint8_t *q_codes, *q_sf, *k_codes, *k_sf, *v_codes, *v_sf;
    PartsPtr out;
    int64_t os[3];
    float* lse;                     // optional fp32 [B][Hq][Nq]; nullptr if not wanted
    const float* qkm;               // fp32 [B][Hq][Nq_p] from the pre-pass
    int* status;                    // the attention kernel's status word
    // accumulator state carried between calls (all nullptr: none); fp32, unnormalized O [B][Hq][Nq][D], m [B][Hq][Nq], l [B][Hq][Nq][2]
    const float *carry_o_in, *carry_m_in, *carry_l_in;
    float *carry_o_out, *carry_m_out, *carry_l_out;
    int causal_shift;               // key j visible to query i iff j <= i + causal_shift (Nk - Nq unless the caller offsets it)
    const int* prepass_status;      // the pre-pass's status word (non-zero: the workspace is incomplete, do nothing)
    const int *cu_q, *cu_k;         // packed variable-length sequences, as in PrepassArgs (nullptr: uniform lengths)
#ifdef SAGE3_DEV_TRACE
    float* debug;                   // development dump of the first CTA; nullptr in normal use
#endif
};

// Encodes a tensor map over a byte tensor [n2][n1][n0] (n0 contiguous) with box [1][b1][b0]; swizzle: 0 none, 1 32 B, 2 64 B,
// 3 128 B.  Returns 0, or the driver's error code (-1: the driver entry point could not be resolved).
int encode_tiled_bytes(void* map64, const void* base, uint64_t n0, uint64_t n1, uint64_t n2, uint32_t b0, uint32_t b1, int swizzle);

cudaError_t launch_prepass(const PrepassArgs& a, cudaStream_t st);
// returns cudaSuccess, or an error; `driver_rc` receives a CUresult when tensor-map encoding failed
cudaError_t launch_attn(const AttnArgs& a, cudaStream_t st, int* driver_rc);

}  // namespace sage3
