/* CPU oracle for the BCPNN layer train-step path -- TEST INFRASTRUCTURE ONLY.
 * Instantiates bcpnn_oracle_impl.h for float (suffix _f32) and double (_f64).
 * Build: see oracle/build.py (gcc -O3 -fopenmp -ffp-contract=off, no fast-math). */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define REAL float
#define FN(name) CAT(name, _f32)
#define EXP expf
#define LOG logf
#include "bcpnn_oracle_impl.h"
#undef REAL
#undef FN
#undef EXP
#undef LOG

#define REAL double
#define FN(name) CAT(name, _f64)
#define EXP exp
#define LOG log
#include "bcpnn_oracle_impl.h"
#undef REAL
#undef FN
#undef EXP
#undef LOG
