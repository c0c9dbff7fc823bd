// Test infrastructure (not product code): prints NVIDIA's own host-side definitions of the narrow formats the layer
// uses, so that the tests can pin the oracle's E2M1 / E4M3 decoders, the nibble order of a packed FP4 byte and the
// round-to-nearest-even encoders against a definition the oracle's author did not write.  Uses only the public
// conversion functions of cuda_fp4.h / cuda_fp8.h, compiled for the host.
//
//   nvcc -o oracle/_build/nv_formats oracle/nv_formats.cpp
//
// Output, one record per line:
//   fp4  <byte> <value of the low nibble> <value of the high nibble>
//   fp8  <byte> <value>                       (E4M3, "nan" for the two NaN codes)
//   q4   <float as hex bits> <nibble>         (float -> E2M1, round to nearest even, saturating)
//   q8   <float as hex bits> <byte>           (float -> E4M3, round to nearest even, saturating to +-448)
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>

static float half_bits_to_float(unsigned short bits) {
  __half h;
  std::memcpy(&h, &bits, sizeof bits);
  return __half2float(h);
}

int main() {
  for (int b = 0; b < 256; ++b) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(b), __NV_E2M1);
    std::printf("fp4 %d %.9g %.9g\n", b, half_bits_to_float(h.x), half_bits_to_float(h.y));
  }
  for (int b = 0; b < 256; ++b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
    const float v = half_bits_to_float(h.x);
    if (std::isnan(v)) std::printf("fp8 %d nan\n", b);
    else std::printf("fp8 %d %.9g\n", b, v);
  }
  // encoders on a grid that contains every rounding boundary of both formats, their neighbours and out-of-range values
  uint32_t state = 12345u;
  for (int i = 0; i < 6000; ++i) {
    float x;
    if (i < 2000) x = (i - 1000) * 0.0078125f;                       // -7.8 .. 7.8 in steps of 2^-7: all E2M1 ties
    else if (i < 4000) x = (i - 3000) * 0.5f;                        // -500 .. 500: E4M3 range and saturation
    else {
      state = state * 1664525u + 1013904223u;
      const uint32_t bits = (state & 0x807FFFFFu) | (((state >> 23) % 24 + 112u) << 23);   // 2^-15 .. 2^8, random mantissa
      std::memcpy(&x, &bits, sizeof x);
    }
    uint32_t xb;
    std::memcpy(&xb, &x, sizeof xb);
    std::printf("q4 %08x %d\n", xb, static_cast<int>(__nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest)));
    std::printf("q8 %08x %d\n", xb, static_cast<int>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)));
  }
  return 0;
}
