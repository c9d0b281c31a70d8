// Replacement for the reference's nt/types/float128.h (its own software binary128, which pulls in a large part of
// nt/bit and nt/math): the matmult path under test never touches a float128 value, the type only has to exist for the
// specialisations that name it.
#ifndef NT_TYPES_FLOAT128_ENSURE_H__
#define NT_TYPES_FLOAT128_ENSURE_H__
#include "../utils/type_traits.h"
namespace nt {
struct float128_t {
    __float128 v;
    constexpr float128_t() : v(0) {}
    constexpr float128_t(double d) : v(d) {}
    constexpr operator double() const { return double(v); }
};
namespace type_traits {
template <> struct is_floating_point<float128_t> : true_type {};
}
}  // namespace nt
#endif
