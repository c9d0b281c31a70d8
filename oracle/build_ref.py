"""Builds oracle/_ref/libntref.so: the REFERENCE's own matmult kernel sources, compiled here, as a second opinion on
the restatement in oracle.cpp.  Test infrastructure only (tests/ and the CPU-baseline leg of bench.py may load it).

    python oracle/build_ref.py [reference root]        (default: $NT_REFERENCE_ROOT, else the checkout beside this repository)

What is compiled: the reference's nt_matmult<T> template (nt/functional/cpu/matmult/nt_matmult.hpp: packing, K-tile
loop, tile schedule), its microkernel (nt_matmult_simde.hpp) and its per-dtype SIMD traits
(nt/mp/simde_traits/simde_traits_avx.h, simde_traits_avx2.h), together with the small type headers they include.  The
files are COPIED from the reference tree into oracle/_ref/src at build time (nothing of the reference is committed in
this repository) and compiled against stand-ins, committed under oracle/ref_shim/, for the three things the reference
includes but does not vendor:
  * SIMD Everywhere (simde): on an AVX2 + FMA + F16C host every simde_mm* function is an alias of the Intel intrinsic
    of the same name; the alias header is generated here from the identifiers the copied sources use.  The handful of
    SVML functions (exp, sin, ... and integer remainder) that GCC's headers lack get scalar loops: matmult uses none.
  * oneTBB: ranges plus a parallel_for that runs the body on the calling thread (TBB only schedules output tiles).
  * half / simde-f16 and the reference's software float128: replaced by _Float16 and a placeholder struct.
The build is skipped (returns None) when the reference tree is absent, as on a GPU box: there the prebuilt library,
which travels with the repository snapshot, is used.
"""
import os
import re
import shutil
import subprocess
import sys

DEFAULT_REFERENCE = os.environ.get("NT_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SHIM = os.path.join(HERE, "ref_shim")
LIB = os.path.join(OUT, "libntref.so")

COPY = [
    "nt/functional/cpu/matmult/nt_matmult.hpp", "nt/functional/cpu/matmult/nt_matmult_simde.hpp",
    "nt/functional/cpu/matmult/nt_matmult_macros.h", "nt/functional/cpu/matmult/nt_matmult_blocks.h",
    "nt/functional/cpu/matmult/nt_matmult.h",
    "nt/mp/simde_traits.h", "nt/mp/simde_traits/simde_traits_avx.h", "nt/mp/simde_traits/simde_traits_avx2.h",
    "nt/types/Types.h", "nt/types/uint_bool.h", "nt/types/complex.h", "nt/types/bit_128_integer.h",
    "nt/utils/type_traits.h", "nt/utils/always_inline_macro.h", "nt/convert/floating.h",
]
REPLACED = {"nt/types/float16.h": "types/float16.h", "nt/types/float128.h": "types/float128.h"}

# SVML-style functions GCC's <immintrin.h> does not have; matmult never calls them, they only have to compile.
UNARY = ["exp", "log", "sin", "cos", "tan", "sinh", "cosh", "tanh", "asin", "acos", "atan", "asinh", "acosh", "atanh"]

DRIVER = r'''
#include <cstdint>
#include "nt/functional/cpu/matmult/nt_matmult.hpp"
// one static pack-buffer pair and one explicit instantiation per dtype, exactly as the reference's
// nt_matmult_<dtype>.cpp files do (e.g. nt_matmult_float16.cpp)
namespace nt::functional::cpu {
_NT_MATMULT_DECLARE_STATIC_BLOCK_(float)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(double)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(float16_t)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(int8_t)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(uint8_t)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(int16_t)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(int32_t)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(int64_t)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(complex_32)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(complex_64)
_NT_MATMULT_DECLARE_STATIC_BLOCK_(complex_128)
}
using namespace nt::functional::cpu;
extern "C" int ntref_matmult(int code, const void* A, const void* B, void* C, int64_t ar, int64_t ac, int64_t br, int64_t bc, int ta, int tb) {
    switch (code) {   // same dtype codes as oracle.cpp / ntb200_dtype
        case 0: nt_matmult<float>((const float*)A, (const float*)B, (float*)C, ar, ac, br, bc, ta, tb); return 0;
        case 1: nt_matmult<nt::float16_t>((const nt::float16_t*)A, (const nt::float16_t*)B, (nt::float16_t*)C, ar, ac, br, bc, ta, tb); return 0;
        case 3: nt_matmult<int8_t>((const int8_t*)A, (const int8_t*)B, (int8_t*)C, ar, ac, br, bc, ta, tb); return 0;
        case 4: nt_matmult<int16_t>((const int16_t*)A, (const int16_t*)B, (int16_t*)C, ar, ac, br, bc, ta, tb); return 0;
        case 5: nt_matmult<int32_t>((const int32_t*)A, (const int32_t*)B, (int32_t*)C, ar, ac, br, bc, ta, tb); return 0;
        case 6: nt_matmult<int64_t>((const int64_t*)A, (const int64_t*)B, (int64_t*)C, ar, ac, br, bc, ta, tb); return 0;
        case 7: nt_matmult<double>((const double*)A, (const double*)B, (double*)C, ar, ac, br, bc, ta, tb); return 0;
        case 8: nt_matmult<uint8_t>((const uint8_t*)A, (const uint8_t*)B, (uint8_t*)C, ar, ac, br, bc, ta, tb); return 0;
        case 11: nt_matmult<nt::complex_64>((const nt::complex_64*)A, (const nt::complex_64*)B, (nt::complex_64*)C, ar, ac, br, bc, ta, tb); return 0;
        case 12: nt_matmult<nt::complex_128>((const nt::complex_128*)A, (const nt::complex_128*)B, (nt::complex_128*)C, ar, ac, br, bc, ta, tb); return 0;
        case 13: nt_matmult<nt::complex_32>((const nt::complex_32*)A, (const nt::complex_32*)B, (nt::complex_32*)C, ar, ac, br, bc, ta, tb); return 0;
    }
    return 1;
}
'''


def alias_header(src_root):
    names = set()
    for dirpath, _, files in os.walk(src_root):
        for f in files:
            text = open(os.path.join(dirpath, f), errors="replace").read()
            names.update(re.findall(r"\bsimde_x?_?mm(?:256|512)?_[a-z0-9_]+\b", text))
            names.update(re.findall(r"\bSIMDE_[A-Z0-9_]+\b", text))
    out = ["// generated by oracle/build_ref.py from the identifiers the copied reference sources use", "#pragma once",
           "#include <immintrin.h>", "#include <cmath>", "#include <cstdint>", "#include <cstring>",
           "#define SIMDE_ARCH_X86_AVX 1", "#define SIMDE_ARCH_X86_AVX2 1", "#define SIMDE_X86_FMA 1", "#define SIMDE_ARCH_SSE3 1",
           "#define SIMDE_FLOAT16_IS_SCALAR 1",
           "typedef __m128 simde__m128; typedef __m128i simde__m128i; typedef __m128d simde__m128d;",
           "typedef __m256 simde__m256; typedef __m256i simde__m256i; typedef __m256d simde__m256d;"]
    # scalar-loop stand-ins
    out.append("""
#define NTREF_UNARY(fn) \\
static inline __m256 ntref_mm256_##fn##_ps(__m256 v) { float t[8]; _mm256_storeu_ps(t, v); for (int i = 0; i < 8; ++i) t[i] = std::fn(t[i]); return _mm256_loadu_ps(t); } \\
static inline __m256d ntref_mm256_##fn##_pd(__m256d v) { double t[4]; _mm256_storeu_pd(t, v); for (int i = 0; i < 4; ++i) t[i] = std::fn(t[i]); return _mm256_loadu_pd(t); } \\
static inline __m128 ntref_mm_##fn##_ps(__m128 v) { float t[4]; _mm_storeu_ps(t, v); for (int i = 0; i < 4; ++i) t[i] = std::fn(t[i]); return _mm_loadu_ps(t); } \\
static inline __m128d ntref_mm_##fn##_pd(__m128d v) { double t[2]; _mm_storeu_pd(t, v); for (int i = 0; i < 2; ++i) t[i] = std::fn(t[i]); return _mm_loadu_pd(t); }
""")
    for fn in UNARY:
        out.append("NTREF_UNARY(%s)" % fn)
    out.append("""
static inline __m256 ntref_mm256_pow_ps(__m256 a, __m256 b) { float x[8], y[8]; _mm256_storeu_ps(x, a); _mm256_storeu_ps(y, b); for (int i = 0; i < 8; ++i) x[i] = std::pow(x[i], y[i]); return _mm256_loadu_ps(x); }
static inline __m256d ntref_mm256_pow_pd(__m256d a, __m256d b) { double x[4], y[4]; _mm256_storeu_pd(x, a); _mm256_storeu_pd(y, b); for (int i = 0; i < 4; ++i) x[i] = std::pow(x[i], y[i]); return _mm256_loadu_pd(x); }
static inline __m128 ntref_mm_pow_ps(__m128 a, __m128 b) { float x[4], y[4]; _mm_storeu_ps(x, a); _mm_storeu_ps(y, b); for (int i = 0; i < 4; ++i) x[i] = std::pow(x[i], y[i]); return _mm_loadu_ps(x); }
static inline __m128d ntref_mm_pow_pd(__m128d a, __m128d b) { double x[2], y[2]; _mm_storeu_pd(x, a); _mm_storeu_pd(y, b); for (int i = 0; i < 2; ++i) x[i] = std::pow(x[i], y[i]); return _mm_loadu_pd(x); }
static inline __m256 ntref_mm256_invsqrt_ps(__m256 v) { return _mm256_div_ps(_mm256_set1_ps(1.f), _mm256_sqrt_ps(v)); }
static inline __m256d ntref_mm256_invsqrt_pd(__m256d v) { return _mm256_div_pd(_mm256_set1_pd(1.0), _mm256_sqrt_pd(v)); }
static inline __m128 ntref_mm_invsqrt_ps(__m128 v) { return _mm_div_ps(_mm_set1_ps(1.f), _mm_sqrt_ps(v)); }
static inline __m128d ntref_mm_invsqrt_pd(__m128d v) { return _mm_div_pd(_mm_set1_pd(1.0), _mm_sqrt_pd(v)); }
#define NTREF_REM(bits, T, n, V, pre) \\
static inline V ntref_##pre##_rem_epi##bits(V a, V b) { T x[n], y[n]; pre##_storeu_si##SZ((V*)x, a); return a; }
static inline __m256i ntref_mm256_rem_epi32(__m256i a, __m256i b) { int32_t x[8], y[8]; _mm256_storeu_si256((__m256i*)x, a); _mm256_storeu_si256((__m256i*)y, b); for (int i = 0; i < 8; ++i) x[i] = y[i] ? x[i] % y[i] : 0; return _mm256_loadu_si256((__m256i*)x); }
static inline __m256i ntref_mm256_rem_epi64(__m256i a, __m256i b) { int64_t x[4], y[4]; _mm256_storeu_si256((__m256i*)x, a); _mm256_storeu_si256((__m256i*)y, b); for (int i = 0; i < 4; ++i) x[i] = y[i] ? x[i] % y[i] : 0; return _mm256_loadu_si256((__m256i*)x); }
static inline __m128i ntref_mm_rem_epi32(__m128i a, __m128i b) { int32_t x[4], y[4]; _mm_storeu_si128((__m128i*)x, a); _mm_storeu_si128((__m128i*)y, b); for (int i = 0; i < 4; ++i) x[i] = y[i] ? x[i] % y[i] : 0; return _mm_loadu_si128((__m128i*)x); }
static inline __m128i ntref_mm_rem_epi64(__m128i a, __m128i b) { int64_t x[2], y[2]; _mm_storeu_si128((__m128i*)x, a); _mm_storeu_si128((__m128i*)y, b); for (int i = 0; i < 2; ++i) x[i] = y[i] ? x[i] % y[i] : 0; return _mm_loadu_si128((__m128i*)x); }
static inline __m256i ntref_mm256_cvtpd_epi64(__m256d v) { double t[4]; int64_t r[4]; _mm256_storeu_pd(t, v); for (int i = 0; i < 4; ++i) r[i] = (int64_t)std::nearbyint(t[i]); return _mm256_loadu_si256((__m256i*)r); }
static inline __m128i ntref_mm_cvtpd_epi64(__m128d v) { double t[2]; int64_t r[2]; _mm_storeu_pd(t, v); for (int i = 0; i < 2; ++i) r[i] = (int64_t)std::nearbyint(t[i]); return _mm_loadu_si128((__m128i*)r); }
static inline __m128d ntref_mm_cvtepi64_pd(__m128i v) { int64_t t[2]; double r[2]; _mm_storeu_si128((__m128i*)t, v); for (int i = 0; i < 2; ++i) r[i] = (double)t[i]; return _mm_loadu_pd(r); }
static inline __m256d ntref_mm256_cvtepi64_pd(__m256i v) { int64_t t[4]; double r[4]; _mm256_storeu_si256((__m256i*)t, v); for (int i = 0; i < 4; ++i) r[i] = (double)t[i]; return _mm256_loadu_pd(r); }
static inline __m256 ntref_mm256_floor_ps(__m256 v) { return _mm256_round_ps(v, _MM_FROUND_FLOOR); }
static inline __m256 ntref_mm256_ceil_ps(__m256 v) { return _mm256_round_ps(v, _MM_FROUND_CEIL); }
static inline __m256d ntref_mm256_floor_pd(__m256d v) { return _mm256_round_pd(v, _MM_FROUND_FLOOR); }
static inline __m256d ntref_mm256_ceil_pd(__m256d v) { return _mm256_round_pd(v, _MM_FROUND_CEIL); }
static inline __m128 ntref_mm_floor_ps(__m128 v) { return _mm_round_ps(v, _MM_FROUND_FLOOR); }
static inline __m128 ntref_mm_ceil_ps(__m128 v) { return _mm_round_ps(v, _MM_FROUND_CEIL); }
static inline __m128d ntref_mm_floor_pd(__m128d v) { return _mm_round_pd(v, _MM_FROUND_FLOOR); }
static inline __m128d ntref_mm_ceil_pd(__m128d v) { return _mm_round_pd(v, _MM_FROUND_CEIL); }
#define NTREF_IDIV(name, T, n256) \
static inline __m256i ntref_mm256_div_##name(__m256i a, __m256i b) { T x[n256], y[n256]; _mm256_storeu_si256((__m256i*)x, a); _mm256_storeu_si256((__m256i*)y, b); for (int i = 0; i < n256; ++i) x[i] = y[i] ? T(x[i] / y[i]) : T(0); return _mm256_loadu_si256((__m256i*)x); } \
static inline __m128i ntref_mm_div_##name(__m128i a, __m128i b) { T x[n256 / 2], y[n256 / 2]; _mm_storeu_si128((__m128i*)x, a); _mm_storeu_si128((__m128i*)y, b); for (int i = 0; i < n256 / 2; ++i) x[i] = y[i] ? T(x[i] / y[i]) : T(0); return _mm_loadu_si128((__m128i*)x); }
NTREF_IDIV(epi8, int8_t, 32) NTREF_IDIV(epu8, uint8_t, 32) NTREF_IDIV(epi16, int16_t, 16) NTREF_IDIV(epu16, uint16_t, 16)
NTREF_IDIV(epi32, int32_t, 8) NTREF_IDIV(epu32, uint32_t, 8) NTREF_IDIV(epi64, int64_t, 4) NTREF_IDIV(epu64, uint64_t, 4)
static inline __m128 ntref_x_mm_round_ps(__m128 v, int mode) { (void)mode; return _mm_round_ps(v, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }
""".replace("#define NTREF_REM(bits, T, n, V, pre) \\\nstatic inline V ntref_##pre##_rem_epi##bits(V a, V b) { T x[n], y[n]; pre##_storeu_si##SZ((V*)x, a); return a; }\n", ""))
    stubbed = set()
    for w in ("mm256", "mm"):
        for fn in UNARY + ["pow", "invsqrt"]:
            for t in ("ps", "pd"):
                stubbed.add("simde_%s_%s_%s" % (w, fn, t))
        for t in ("rem_epi32", "rem_epi64", "cvtpd_epi64", "cvtepi64_pd"):
            stubbed.add("simde_%s_%s" % (w, t))
    stubbed.add("simde_x_mm_round_ps")
    for w in ("mm256", "mm"):
        for fn in ("floor", "ceil"):
            for t in ("ps", "pd"):
                stubbed.add("simde_%s_%s_%s" % (w, fn, t))
        for t in ("epi8", "epu8", "epi16", "epu16", "epi32", "epu32", "epi64", "epu64"):
            stubbed.add("simde_%s_div_%s" % (w, t))
            for cmp in ("cmpgt", "cmpeq"):           # some of these names are only formed by token pasting in the sources
                if t.startswith("epi"):
                    names.add("simde_%s_%s_%s" % (w, cmp, t))
    names.update(stubbed)
    for n in sorted(names):
        if n.startswith("SIMDE_"):
            if n in ("SIMDE_ARCH_X86_AVX", "SIMDE_ARCH_X86_AVX2", "SIMDE_X86_FMA", "SIMDE_ARCH_SSE3", "SIMDE_FLOAT16_IS_SCALAR"):
                continue
            if n.startswith("SIMDE_MM_FROUND") or n.startswith("SIMDE_CMP_") or n == "SIMDE_MM_SHUFFLE":
                out.append("#define %s %s" % (n, n[len("SIMDE"):]))          # SIMDE_MM_FROUND_x -> _MM_FROUND_x, SIMDE_CMP_x -> _CMP_x
            continue
        if n in stubbed:
            out.append("#define %s ntref_%s" % (n, n[len("simde_"):]))
        else:
            out.append("#define %s _%s" % (n, n[len("simde_"):]))
    return "\n".join(out) + "\n"


def build(reference=None, force=False):
    reference = reference or DEFAULT_REFERENCE
    if not os.path.isdir(os.path.join(reference, "nt")):
        return LIB if os.path.exists(LIB) else None
    if os.path.exists(LIB) and not force:
        return LIB
    src = os.path.join(OUT, "src")
    if os.path.exists(src):
        shutil.rmtree(src)
    for rel in COPY:
        dst = os.path.join(src, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(reference, rel), dst)
    for rel, shim in REPLACED.items():
        shutil.copyfile(os.path.join(SHIM, shim), os.path.join(src, rel))
    gen = os.path.join(OUT, "gen")
    os.makedirs(gen, exist_ok=True)
    with open(os.path.join(gen, "ntref_simde_alias.h"), "w") as f:
        f.write(alias_header(src))
    with open(os.path.join(gen, "driver.cpp"), "w") as f:
        f.write(DRIVER)
    cmd = ["g++", "-std=c++17", "-O3", "-march=x86-64-v3", "-mf16c", "-fPIC", "-shared", "-w", "-fpermissive", "-I", gen, "-I", SHIM, "-I", src,
           os.path.join(gen, "driver.cpp"), "-o", LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stderr[-6000:])
        raise RuntimeError("the reference's matmult sources did not compile against the stand-in headers")
    return LIB


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
