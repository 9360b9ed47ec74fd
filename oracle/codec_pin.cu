// Known-answer generator for the two number formats on the SageAttention3 path.
//
// TEST INFRASTRUCTURE ONLY.  Runs on the host (no GPU needed): it calls NVIDIA's own host-side
// converters from cuda_fp4.h / cuda_fp8.h -- the same conversions the reference performs on device
// with `cvt.rn.satfinite.e2m1x2.f32` (sageattn3/quantization/fp4_quantization_4d.cu:86-89) and
// `__nv_fp8_e4m3(float)` (fp4_quantization_4d.cu:199-202) -- on a fixed sweep of inputs and prints
// "x_bits e2m1_code e4m3_byte" lines.  oracle/make_codec_pin.py turns the output into
// tests/golden/codec_pin.npz, against which the Python oracle's codecs are checked.
//
// Build + run:  nvcc -o oracle/_ref/codec_pin oracle/codec_pin.cu && oracle/_ref/codec_pin
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cstdint>
#include <cstdio>
#include <cstring>

static void emit(float x) {
    uint32_t bits;
    std::memcpy(&bits, &x, 4);
    unsigned c4 = __nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest) & 0xF;
    unsigned c8 = __nv_cvt_float_to_fp8(x < 0 ? -x : x, __NV_SATFINITE, __NV_E4M3) & 0xFF;
    std::printf("%u %u %u\n", bits, c4, c8);
}

int main() {
    // 1. a dense linear sweep through the E2M1 range, both signs, with all tie points hit exactly
    for (int i = -7 * 64; i <= 7 * 64; ++i) emit(i / 64.0f);
    // 2. neighbours (one fp32 ulp either side) of every E2M1 and E4M3 rounding boundary
    const float ties4[] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f, 6.0f};
    for (float t : ties4)
        for (int s = -1; s <= 1; s += 2) {
            uint32_t b; float x = s * t; std::memcpy(&b, &x, 4);
            for (int d = -1; d <= 1; ++d) { uint32_t bb = b + d; float y; std::memcpy(&y, &bb, 4); emit(y); }
        }
    // 3. every E4M3 value, the midpoint to its successor, and that midpoint's fp32 neighbours
    for (int code = 0; code < 0x7E; ++code) {
        __half_raw h0 = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code, __NV_E4M3);
        __half_raw h1 = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(code + 1), __NV_E4M3);
        float a = __half2float(__half(h0)), b = __half2float(__half(h1));
        float mid = 0.5f * (a + b);
        uint32_t mb; std::memcpy(&mb, &mid, 4);
        emit(a);
        for (int d = -1; d <= 1; ++d) { uint32_t bb = mb + d; float y; std::memcpy(&y, &bb, 4); emit(y); }
    }
    // 4. saturation and tiny values
    const float extra[] = {448.f, 449.f, 464.f, 465.f, 480.f, 1000.f, 1e6f, 3.0e38f, 1e-3f, 9.765625e-4f,
                           9.7656256e-4f, 9.76e-4f, 1e-5f, 1e-10f, 0.f, 6.5f, 7.f, 100.f, -100.f};
    for (float x : extra) emit(x);
    // 5. a pseudo-random log-uniform sweep (LCG) over [2^-12, 2^10]
    uint32_t s = 12345u;
    for (int i = 0; i < 20000; ++i) {
        s = s * 1664525u + 1013904223u;
        int e = (int)((s >> 8) % 22) - 12;
        s = s * 1664525u + 1013904223u;
        float m = 1.0f + (s >> 9) * (1.0f / 8388608.0f);
        float x = std::ldexp(m, e);
        if (s & 256u) x = -x;
        emit(x);
    }
    return 0;
}
