// Host-callable launchers of the pointwise kernels (elementwise.cu) and the reductions / index kernels
// (reduce.cu).  All launches go to the given stream and never synchronise.
#pragma once
#include "common.cuh"

namespace cgk {

enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_F8 = 3, DT_U32 = 4 };  // = cg::Dtype
enum { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_LT, B_GT, B_GTE, B_LTE, B_EQ };  // = cg::BinOp
enum { U_NEG = 0, U_SIN, U_COS, U_EXP, U_LOG, U_FLOOR, U_ROUND };                // = cg::UnOp

// `vec` > 1 selects the 16-byte vector path; the caller guarantees its preconditions (inner extent a
// multiple of the vector width, every operand's inner stride 1 or 0, 16-byte aligned bases and outer strides).
int vector_width(int elem_size_in, int elem_size_out);
void launch_binary(int op, int dtype, const View4& vw, int vec, const void* a, const void* b, void* o, unsigned* err,
                   int sm_count, cudaStream_t st);
void launch_unary(int op, int dtype, const View4& vw, int vec, const void* a, void* o, int sm_count, cudaStream_t st);
void launch_where(int dtype, const View4& vw, int vec, const void* m, const void* x, const void* y, void* o,
                  int sm_count, cudaStream_t st);
void launch_copy(int elem_size, const View4& vw, int vec, const void* a, void* o, int sm_count, cudaStream_t st);
void launch_cast(int dt_in, int dt_out, const View4& vw, int vec, const void* a, void* o, int sm_count,
                 cudaStream_t st);
void launch_arange(unsigned* o, long long n, int sm_count, cudaStream_t st);

// ---- reduce.cu ------------------------------------------------------------------------------
enum { R_SUM = 0, R_MAX = 1, R_ARGMAX = 2 };
// Rows of `n` elements: row r starts at a + row_offset(r) where the outer index space is vw (rank-1 dims,
// strides in vw.sa) and the inner stride is `inner_stride`.  Output is contiguous [rows].
void launch_argmax_two_stage(int dtype, const void* x, long long row_stride, long long rows, long long n, void* scratch,
                             unsigned* out, cudaStream_t st);
void launch_reduce(int kind, int dtype, const View4& outer, long long rows, long long n, long long inner_stride,
                   const void* a, void* o, int sm_count, cudaStream_t st);
// out = softmax over the last axis of contiguous x [rows, n] (f32, bf16 or f16): the nn::softmax graph in one kernel.
void launch_softmax(int dtype, const void* x, void* out, long long rows, long long n, cudaStream_t st);
// out[o, j, i] = x[o, idx[j], i]; x is contiguous [outer, dim, inner]; idx has n_idx entries (stride idx_stride).
void launch_gather(int elem_size, const void* x, const unsigned* idx, long long idx_stride, void* out, long long outer,
                   long long dim, long long n_idx, long long inner, unsigned* err, int sm_count, cudaStream_t st);
// values/indices of the k largest per contiguous row (stable: equal values keep ascending index order).
void launch_topk(int dtype, const void* x, void* values, unsigned* indices, long long rows, long long n, long long k,
                 cudaStream_t st);
// *flag |= 1 if any element is > 0 (floats) / != 0 (u32); contiguous input.
void launch_any_positive(int dtype, const void* x, long long n, unsigned* flag, int sm_count, cudaStream_t st);
// *flag |= 1 if any element pair differs (NaN differs from everything); contiguous inputs.
void launch_any_diff(int dtype, const void* a, const void* b, long long n, unsigned* flag, int sm_count,
                     cudaStream_t st);

}  // namespace cgk
