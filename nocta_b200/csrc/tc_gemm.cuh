// Host-side interface of the tcgen05 / TMEM / TMA contraction kernels (tc_gemm.cu).
#pragma once
#include "nc_common.cuh"

namespace tc {

// D(M,N) row-major (ldd) = alpha * A * B^T + beta * D + bias[n].
//   a_mn == false: A stored (M,K) row-major, lda;  a_mn == true: A stored (K,M) row-major, lda.
//   b_mn == false: B stored (N,K) row-major, ldb;  b_mn == true: B stored (K,N) row-major, ldb.
// mode: NC_CUDA_MATH_TF32 / _TF32_RNA / _3XTF32.
// Returns NC_CUDA_ERR_UNSUPPORTED (without setting the sticky status) when the operands cannot be
// described to TMA (alignment, leading dimensions) or the problem is too small to be worth a
// 128-row tile; the caller then uses the SIMT kernel.
int gemm(float* D, int ldd, const float* A, int lda, bool a_mn, const float* B, int ldb, bool b_mn, int M, int N,
         int K, const float* bias, float alpha, float beta, int mode, cudaStream_t st);

// Channels-last implicit-GEMM convolution, stride 1:
//   y(N,Ho,Wo,Cout) = conv(x(N,H,W,Cin), wpacked) + bias,  Ho = H + 2*pad - kH + 1.
// wpacked is (kH, kW, Cout, Cin) dense — see pack_weights_*.
int conv_nhwc(float* y, const float* x, const float* wpacked, const float* bias, int N, int H, int W, int Cin,
              int Cout, int kH, int kW, int pad, int mode, cudaStream_t st);

// dW partials for a stride-1 channels-last convolution and their ordered reduction into the
// reference weight layout (Cout, Cin, kH, kW).
int conv_dw_nhwc(float* dW, const float* dy, const float* x, int N, int H, int W, int Cin, int Cout, int kH, int kW,
                 int pad, int mode, cudaStream_t st);

// Halo-resident kernels (tc_conv.cu), plain TF32 mode, stride 1, filters up to 3 x 3; NC_CUDA_ERR_UNSUPPORTED otherwise.
//   conv_halo_nhwc:    forward / input gradient with the activation halo of a pixel tile resident in shared memory
//   conv_dw_halo_nhwc: weight gradient with one dY tile and one x halo tile serving all filter taps of a row
int conv_halo_nhwc(float* y, const float* x, const float* wpacked, const float* bias, int N, int H, int W, int Cin, int Cout,
                   int kH, int kW, int pad, int mode, cudaStream_t st);
int conv_dw_halo_nhwc(float* dW, const float* dy, const float* x, int N, int H, int W, int Cin, int Cout, int kH, int kW,
                      int pad, int mode, cudaStream_t st);
// partial[z][co][(kh*kW+kw)*Cin + ci] summed over z in order -> dW (Cout, Cin, kH, kW)
int dw_reduce(float* dW, const float* partial, int splits, int Cout, int Cin, int kH, int kW, cudaStream_t st);

// (Cout,Cin,kH,kW) -> (kH,kW,Cout,Cin) for the forward; -> flipped (kH,kW,Cin,Cout) for dX.
int pack_weights_fwd(float* wp, const float* w, int Cout, int Cin, int kH, int kW, bool round, cudaStream_t st);
int pack_weights_dx(float* wp, const float* w, int Cout, int Cin, int kH, int kW, bool round, cudaStream_t st);

}  // namespace tc
