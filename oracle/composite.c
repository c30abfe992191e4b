/*
 * CPU restatement of the compositing kernels, float and double instantiations.
 * TEST INFRASTRUCTURE ONLY (see oracle/__init__.py); built into oracle/_build/liboracle.so by
 * oracle/Makefile and loaded through ctypes by oracle/composite.py.
 */
#include <math.h>

#define REAL float
#define FN(name) name##_f32
#define EXP expf
#define FMOD fmodf
#include "composite_impl.h"
#undef REAL
#undef FN
#undef EXP
#undef FMOD

#define REAL double
#define FN(name) name##_f64
#define EXP exp
#define FMOD fmod
#include "composite_impl.h"
#undef REAL
#undef FN
#undef EXP
#undef FMOD
