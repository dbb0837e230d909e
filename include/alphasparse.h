#pragma once
/*
 * Umbrella header of the B200 (sm_100a) CUDA backend for the CSR mv/mm path of the
 * AlphaSparse C API.  A program written against the reference's <alphasparse.h>
 * (include/alphasparse.h:1-33 of the reference) compiles unchanged against this one for the
 * entry points declared here: handles built from CSR or COO arrays, alphasparse_?_mv and
 * alphasparse_?_mm.  Enum values, struct layouts and calling conventions are identical.
 */
#ifdef __cplusplus
extern "C" {
#endif

#include "alphasparse/types.h"
#include "alphasparse/spdef.h"
#include "alphasparse/spapi.h"
#include "alphasparse/util.h"
#include "alphasparse/spapi_cuda.h"

#ifdef __cplusplus
}
#endif
