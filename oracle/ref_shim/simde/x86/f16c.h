// Stand-in for a header of the SIMD Everywhere library, which the reference includes but does not vendor.  On an
// x86-64 host with AVX2, FMA and F16C every simde_mm* function the reference uses is a 1:1 alias of the Intel
// intrinsic of the same name; the aliases are generated from the reference's own sources at build time.
#pragma once
#include "ntref_simde_alias.h"
