// Host fp8 codecs: E4M3 (finite, max 448, no infinities) and E5M2 (max 57344), round to nearest even, saturating.
// The same conversions as the device quantizers, for CPU oracles and for tools that inspect fp8 tensors
// (counterpart of the reference's include/nanochat/fp8.h).
#include <cmath>
#include <cstdint>
#include <cstring>

#include "core.h"

namespace ncb {

namespace {

// Generic small-float encoder: `ebits` exponent bits, `mbits` mantissa bits, bias, largest finite value.
std::uint8_t Encode(float v, int ebits, int mbits, int bias, float max_finite, std::uint8_t nan_code) {
  std::uint32_t bits;
  std::memcpy(&bits, &v, 4);
  const std::uint8_t sign = static_cast<std::uint8_t>((bits >> 31) << 7);
  if (std::isnan(v)) return static_cast<std::uint8_t>(sign | nan_code);
  float a = std::fabs(v);
  if (a >= max_finite) a = max_finite;  // saturate (also infinities)
  if (a == 0.0f) return sign;
  int e;
  const float fr = std::frexp(a, &e);   // a = fr * 2^e, fr in [0.5, 1)
  int exp = e - 1 + bias;               // biased exponent of the normalised value 1.xxx * 2^(e-1)
  float scaled;
  if (exp >= 1) {
    scaled = (fr * 2.0f - 1.0f) * static_cast<float>(1 << mbits);            // mantissa in units of 2^-mbits
  } else {
    scaled = a / std::ldexp(1.0f, 1 - bias - mbits);                           // subnormal: units of the smallest step
    exp = 0;
  }
  // round to nearest even
  float fl = std::floor(scaled);
  const float rem = scaled - fl;
  if (rem > 0.5f || (rem == 0.5f && (static_cast<int>(fl) & 1))) fl += 1.0f;
  int mant = static_cast<int>(fl);
  if (exp == 0 && mant == (1 << mbits)) {
    exp = 1;
    mant = 0;
  } else if (exp >= 1 && mant == (1 << mbits)) {
    exp += 1;
    mant = 0;
  }
  const int max_exp = (1 << ebits) - 1;
  std::uint8_t code = static_cast<std::uint8_t>((exp << mbits) | mant);
  // saturation was applied on the value, so the code cannot exceed the largest finite code
  (void)max_exp;
  return static_cast<std::uint8_t>(sign | code);
}

float Decode(std::uint8_t c, int ebits, int mbits, int bias, bool ieee_specials) {
  const int sign = c >> 7;
  const int exp = (c >> mbits) & ((1 << ebits) - 1);
  const int mant = c & ((1 << mbits) - 1);
  float v;
  if (ieee_specials && exp == (1 << ebits) - 1) {
    v = mant == 0 ? INFINITY : NAN;
  } else if (!ieee_specials && exp == (1 << ebits) - 1 && mant == (1 << mbits) - 1) {
    v = NAN;  // E4M3: only S.1111.111 is NaN
  } else if (exp == 0) {
    v = std::ldexp(static_cast<float>(mant), 1 - bias - mbits);
  } else {
    v = std::ldexp(1.0f + static_cast<float>(mant) / static_cast<float>(1 << mbits), exp - bias);
  }
  return sign ? -v : v;
}

}  // namespace

std::uint8_t FloatToE4M3(float v) { return Encode(v, 4, 3, 7, 448.0f, 0x7F); }
float E4M3ToFloat(std::uint8_t c) { return Decode(c, 4, 3, 7, false); }
std::uint8_t FloatToE5M2(float v) { return Encode(v, 5, 2, 15, 57344.0f, 0x7F); }
float E5M2ToFloat(std::uint8_t c) { return Decode(c, 5, 2, 15, true); }

}  // namespace ncb

extern "C" {
// format: 0 = E4M3, 1 = E5M2
void ncb_fp8_encode(const float* src, unsigned char* dst, long long n, int format) {
  for (long long i = 0; i < n; ++i) dst[i] = format == 0 ? ncb::FloatToE4M3(src[i]) : ncb::FloatToE5M2(src[i]);
}
void ncb_fp8_decode(const unsigned char* src, float* dst, long long n, int format) {
  for (long long i = 0; i < n; ++i) dst[i] = format == 0 ? ncb::E4M3ToFloat(src[i]) : ncb::E5M2ToFloat(src[i]);
}
}
