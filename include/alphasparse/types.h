#pragma once
/*
 * Scalar and index types of the C ABI.
 * Mirrors include/alphasparse/types.h:43-112 of the reference: 32-bit ALPHA_INT unless the
 * build overrides it, two-float / two-double complex structs, and the (row, col, value)
 * point records the COO->CSR conversion sorts.
 */
#include <stdint.h>
#include <stdbool.h>
#include <stddef.h>

#ifndef ALPHA_INT
#define ALPHA_INT int32_t
#endif
#ifndef ALPHA_INT64
#define ALPHA_INT64 int64_t
#endif

typedef struct { float real;  float imag;  } ALPHA_Complex8;
typedef struct { double real; double imag; } ALPHA_Complex16;

typedef struct { ALPHA_INT x; ALPHA_INT y; float v;  } point_s_t;
typedef struct { ALPHA_INT x; ALPHA_INT y; double v; } point_d_t;
