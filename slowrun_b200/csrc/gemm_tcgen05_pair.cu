// CTA-pair variant of the persistent GEMM: the kernel itself is the template in gemm_pair_kernel.cuh (protocol and
// layout are described there), instantiated here with the plain store epilogue for bf16 operands (every large GEMM of
// the training step) and for fp8 operands (K-major e4m3 / e5m2, fp32 accumulation; the reference reaches cuBLASLt
// through torch._scaled_mm for these, tiny/cuda_kernels.py:345-352).
//
// Same contract as the single-CTA kernel (gemm_tcgen05.cu), symmetric-output mode included (256-row tiles that touch the
// upper triangle are computed, the rest is filled by mirrored stores).
#include "gemm_pair_kernel.cuh"

// CTA-pair GEMM; arguments as sr_gemm_bf16 (gemm_tcgen05.cu). bn in {128, 160, 256} (160 only with a
// K-major B), already chosen by the caller. Returns 0 on successful launch.
extern "C" int sr_gemm_bf16_pair(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                                 long long lda, long long ldb, long long ldc, long long ldcin, long long strideA,
                                 long long strideB, long long strideC, long long strideCin, int a_mn, int b_mn,
                                 int c_fp32, int cin_fp32, float alpha, float beta, const float* alpha_ptr,
                                 const float* row_scale, int sym, int splitk, int bn, int max_ctas, int* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (sym && (M != N || bn == 160)) return -6;
  if (bn != 128 && bn != 160 && bn != 256) return -7;
  if (bn == 160 && b_mn) return -7;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.C = C; p.ldc = ldc; p.strideC = strideC; p.c_fp32 = c_fp32;
  p.Cin = Cin; p.ldcin = ldcin; p.strideCin = strideCin; p.cin_fp32 = cin_fp32;
  p.alpha = alpha; p.beta = beta; p.alpha_ptr = alpha_ptr; p.row_scale = row_scale; p.sym = sym; p.status = status;
  p.splitk = sym ? 0 : splitk;
  CUtensorMap ma, mb;
  int rc;
  if (!a_mn) rc = encode_bf16_map(&ma, A, K, M, batch, lda, strideA, BK, BM);
  else       rc = encode_bf16_map(&ma, A, M, K, batch, lda, strideA, 64, BK);
  if (rc) return rc;
  if (!b_mn) rc = encode_bf16_map(&mb, B, K, N, batch, ldb, strideB, BK, bn / 2);
  else       rc = encode_bf16_map(&mb, B, N, K, batch, ldb, strideB, 64, BK);
  if (rc) return rc - 10;
  if (bn == 256) return launch_pair<256, 2, EpiStore>(ma, mb, p, max_ctas, 1, stream);
  if (bn == 160) return launch_pair<160, 2, EpiStore>(ma, mb, p, max_ctas, 1, stream);
  return launch_pair<128, 2, EpiStore>(ma, mb, p, max_ctas, 1, stream);
}

// out[b] = alpha * A[b] B[b]^T (+ beta * Cin[b]) with fp8 operands stored K-major: A is [M, K], B is [N, K], one byte
// per element, K contiguous, leading dimensions multiples of 16. a_fmt / b_fmt: 0 = e4m3, 1 = e5m2. Scales of a
// per-tensor quantisation go into alpha (or alpha_ptr); accumulation is fp32, the output bf16 or fp32.
extern "C" int sr_gemm_fp8_pair(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K, int batch,
                                long long lda, long long ldb, long long ldc, long long ldcin, long long strideA,
                                long long strideB, long long strideC, long long strideCin, int a_fmt, int b_fmt,
                                int c_fp32, int cin_fp32, float alpha, float beta, const float* alpha_ptr,
                                const float* row_scale, int bn, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (bn == 0) bn = N > 128 ? 256 : 128;
  if (bn != 128 && bn != 256) return -7;
  if ((a_fmt | b_fmt) & ~1) return -2;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.C = C; p.ldc = ldc; p.strideC = strideC; p.c_fp32 = c_fp32;
  p.Cin = Cin; p.ldcin = ldcin; p.strideCin = strideCin; p.cin_fp32 = cin_fp32;
  p.alpha = alpha; p.beta = beta; p.alpha_ptr = alpha_ptr; p.row_scale = row_scale; p.status = status;
  p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  CUtensorMap ma, mb;
  int rc = encode_u8_map(&ma, A, K, M, batch, lda, strideA, 128, BM);
  if (rc) return rc;
  rc = encode_u8_map(&mb, B, K, N, batch, ldb, strideB, 128, bn / 2);
  if (rc) return rc - 10;
  if (bn == 256) return launch_pair<256, 1, EpiStore>(ma, mb, p, max_ctas, 1, stream);
  return launch_pair<128, 1, EpiStore>(ma, mb, p, max_ctas, 1, stream);
}
