// Conventions shared by every extern "C" launcher of the library.
//
// As in the reference (cuda/src/kernels.cu:1040, :5671-5672; src/compute/cuda_ffi.rs:143-1066):
// every launcher returns int, 0 = launched, a positive value = the cudaError_t of the launch,
// a negative value = the call was refused before any launch.  The last argument is a
// cudaStream_t passed as void* (null = default stream); launchers never synchronise and never
// allocate.  All pointers are device pointers owned by the caller.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define VIB3_OK 0
#define VIB3_ERR_UNSUPPORTED (-1)  // the reference's "-1: not available on this GPU / dtype"
#define VIB3_ERR_COUNT (-2)        // the reference's "-2: count out of range"
#define VIB3_ERR_NULL (-3)
#define VIB3_ERR_ALIGN (-4)
#define VIB3_ERR_SHAPE (-5)
#define VIB3_ERR_RANGE (-6)        // row range outside the matrix, page missing
#define VIB3_ERR_STATE (-7)        // pool / planner object in the wrong state
#define VIB3_ERR_CAPACITY (-8)     // request larger than a built-in fixed-size buffer
