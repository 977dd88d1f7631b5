// What the tensor-core matrix product shares with the other tcgen05 kernels of the library.
#pragma once
#include <cuda.h>

// A 2-D tensor map over a row-major bfloat16 matrix [rows, cols] with row pitch `ld` elements:
// box [box_rows, 64], 128-byte swizzle, zero fill out of bounds.  False when the driver
// refuses the map.
bool zi_internal_make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows);

// The device word in which the tcgen05 kernels record a wait that ran out (0: none).
int* zi_internal_status_word();
