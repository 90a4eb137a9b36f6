// Tall-and-skinny fp32 products for block Gram-Schmidt panels (see skinny.cu).
#pragma once
#include <cuda_runtime.h>

namespace hb {

// number of partial products tall_t_mul writes for a contraction length n
int tall_splits(int n);

// C[s][b] = partial X[b]^T W[b] over the s-th part of the n rows; C: [tall_splits(n), batch, m, p] fp32, p <= 32.
cudaError_t launch_tall_t_mul(const float* X, long long ldx, long long strideX, const float* W, long long ldw,
                              long long strideW, int batch, int n, int m, int p, float* C, cudaStream_t stream);

// Inverses of the diagonal blocks of upper-triangular matrices: for T = Q[b] (n x n, row stride ld, batch stride
// strideQ) and block index i, X[b][i] = inverse of T[i*blk : (i+1)*blk, i*blk : (i+1)*blk] (the last block may be
// smaller; it is completed with an identity).  X: [batch, ceil(n / blk), blk, blk] fp32, blk = kTriBlock.
constexpr int kTriBlock = 128;
cudaError_t launch_tri_inv_blocks(const float* Q, long long ld, long long strideQ, int batch, int n, float* X,
                                  cudaStream_t stream);

// Upper Cholesky factor and its inverse of one diagonal leaf (size <= kTriBlock) of a batch of symmetric positive definite
// matrices: G points at the leaf's first element (row stride ldg, batch stride strideG), likewise R; X: the leaf's
// kTriBlock x kTriBlock inverse block per matrix (batch stride strideX), completed with an identity for short leaves.
// info[b] is incremented when a pivot of matrix b was not positive.
cudaError_t launch_chol_inv_leaf(const float* G, long long ldg, long long strideG, float* R, long long ldr, long long strideR,
                                 float* X, long long strideX, int batch, int size, int* info, cudaStream_t stream);

// Row-major upper triangle of square matrices, [batch, n, n] <-> [batch, n (n + 1) / 2]; elements of 2 or 4 bytes are
// moved as bits.  Unpacking writes zeros below the diagonal.  blockIdx.y = batch (<= 65535).
cudaError_t launch_triu_pack(const void* dense, void* line, int elem_bytes, int batch, int n, cudaStream_t stream);
cudaError_t launch_triu_unpack(const void* line, void* dense, int elem_bytes, int batch, int n, cudaStream_t stream);

}  // namespace hb
