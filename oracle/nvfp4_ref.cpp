// TEST INFRASTRUCTURE ONLY - host restatement of the reference's NVFP4 quantiser
// (tools/analysis/nvfp4/primitive.cu:50-75) through the CUDA toolkit's own
// host-callable conversions (__nv_fp8_e4m3, __nv_cvt_float_to_fp4), the same
// functions the reference kernel calls on the device.  Built with g++ by
// oracle/build.py; used only by tests to cross-check oracle/nvfp4.py.
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <math.h>
#include <stdint.h>

static float bf16_bits_to_float(uint16_t b) {
    union { uint32_t u; float f; } c;
    c.u = (uint32_t)b << 16;
    return c.f;
}

extern "C" int oracle_nvfp4_quantize(const uint16_t *input_bf16, uint8_t *packed, uint8_t *scales, float *decoded,
                                     int rows, int k, float tensor_scale) {
    if (k % 16) return 1;
    for (long long g = 0; g < (long long)rows * (k / 16); ++g) {
        float v[16], amax = 0.f;
        for (int i = 0; i < 16; ++i) {
            v[i] = bf16_bits_to_float(input_bf16[g * 16 + i]) / tensor_scale;  // primitive.cu:58
            amax = fmaxf(amax, fabsf(v[i]));                                    // :59-60
        }
        __nv_fp8_e4m3 sf(fmaxf(amax / 6.f, 1.f / 512.f));                       // :62
        const float scale = float(sf);                                          // :63
        uint8_t q[16];
        for (int i = 0; i < 16; ++i)
            q[i] = (uint8_t)__nv_cvt_float_to_fp4(v[i] / scale, __NV_E2M1, cudaRoundNearest) & 0xF;  // :64
        scales[g] = sf.__x;                                                     // :66
        for (int i = 0; i < 8; ++i) packed[g * 8 + i] = q[2 * i] | (q[2 * i + 1] << 4);  // :69-70
        if (decoded)
            for (int i = 0; i < 16; ++i) {
                __half_raw h = __nv_cvt_fp4_to_halfraw(q[i], __NV_E2M1);
                decoded[g * 16 + i] = __half2float(__half(h)) * scale * tensor_scale;    // :71-74
            }
    }
    return 0;
}

extern "C" float oracle_e4m3_to_float(uint8_t bits) {
    __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)bits, __NV_E4M3);
    return __half2float(__half(h));
}

extern "C" uint8_t oracle_float_to_e4m3(float x) { return __nv_fp8_e4m3(x).__x; }

extern "C" uint8_t oracle_float_to_e2m1(float x) {
    return (uint8_t)__nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest) & 0xF;
}
