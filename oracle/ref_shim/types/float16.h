// Replacement for the reference's nt/types/float16.h, which takes its half type from simde-f16.h or from the `half`
// library (neither is vendored).  On this toolchain both amount to an IEEE binary16 value with round-to-nearest-even
// conversions from float, which is what _Float16 is: the matmult traits never compute in this type, they only widen
// it to float (cvtph_ps) and narrow the vector result back (cvtps_ph).
#ifndef _NT_TYPES_FLOAT16_ENSURE_H_
#define _NT_TYPES_FLOAT16_ENSURE_H_
#include <cstdint>
#include <iostream>
#include "../utils/type_traits.h"
#define _HALF_FLOAT_SUPPORT_
namespace nt {
using float16_t = _Float16;
#define _NT_FLOAT16_TO_FLOAT32_(f16) float(f16)
#define _NT_FLOAT32_TO_FLOAT16_(f) ::nt::float16_t(f)
inline std::ostream& operator<<(std::ostream& os, const float16_t& val) { return os << float(val); }
inline int16_t _NT_FLOAT16_TO_INT16_(float16_t fp) noexcept {
    int16_t out;
    __builtin_memcpy(&out, &fp, 2);
    return out;
}
namespace type_traits {
constexpr bool simde_float16 = true;
template <> struct is_floating_point<float16_t> : true_type {};
template <> struct is_floating_point<const float16_t> : true_type {};
template <> struct make_unsigned<float16_t> { using type = uint16_t; };
}  // namespace type_traits
}  // namespace nt
#endif
