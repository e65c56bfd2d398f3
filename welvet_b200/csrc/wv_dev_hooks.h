// Development hooks of libwelvet_cuda.so: exported for the test-suite and for tuning runs, not part
// of the public C ABI (include/welvet_cuda.h) and without a counterpart in the reference.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
// Register-load GEMV: rows per warp / column split / prefetch depth / grid size (0 = built-in choice).
void wv_set_tuning(int rows_per_warp, int col_split, int depth, int grid);
// Bulk-copy-fed kernels: rows per row group per tile (1, 2, 4, 8; 11-14 without register prefetch) or
// 21 / 22 / 24 to route the formats with one parameter group per 32 weights through the tensor-pipe
// kernel; ring depth cap in the low two digits of `stages`, tiles issued ahead of the activation
// loads in the hundreds.
void wv_set_tma_tuning(int rows_per_group, int stages);
// Width of the activation records of the integer-dot kernels: 0 = chosen per launch from the input
// vector (16-bit unless it has isolated outliers), 3 = always 24-bit.
void wv_set_act_width(int limbs);
#ifdef __cplusplus
}
#endif
