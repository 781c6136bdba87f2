/*
 * Stand-in for <libxsmm.h>, TEST INFRASTRUCTURE.
 *
 * The reference's CPU BH4 extension (bh4/cpu/torch_extension.cpp) includes <libxsmm.h> and uses exactly one
 * thing from it: libxsmm_mmfunction<float>, a small-matrix multiply kernel built for fixed (m, n, k) and leading
 * dimensions and called as kernel(a, b, c).  libxsmm is a third-party library that is not part of the reference
 * tree and is not installed here, so this header provides that one class with libxsmm's documented meaning
 * (column-major operands, C += A * B, alpha = beta = 1, no transposes) as plain loops.  It lets the reference's
 * source file compile unmodified into oracle/_ref, where it pins the CPU convention of the projection and is
 * timed as a CPU baseline ("stand-in GEMM": the real library would be faster).  Nothing here comes from libxsmm.
 */
#ifndef LFFN_STANDIN_LIBXSMM_H_
#define LFFN_STANDIN_LIBXSMM_H_

#define LIBXSMM_GEMM_FLAG_NONE 0

template <typename T>
class libxsmm_mmfunction {
  public:
    libxsmm_mmfunction() : m_(0), n_(0), k_(0), lda_(0), ldb_(0), ldc_(0) {}
    libxsmm_mmfunction(int /*flags*/, int m, int n, int k, int lda, int ldb, int ldc)
        : m_(m), n_(n), k_(k), lda_(lda), ldb_(ldb), ldc_(ldc) {}

    /* C[i + j*ldc] += sum_p A[i + p*lda] * B[p + j*ldb]   (column-major, 0 <= i < m, 0 <= j < n, 0 <= p < k) */
    void operator()(const T *a, const T *b, T *c) const {
        for (int j = 0; j < n_; j++) {
            T *cj = c + (long)j * ldc_;
            for (int p = 0; p < k_; p++) {
                const T bpj = b[p + (long)j * ldb_];
                const T *ap = a + (long)p * lda_;
                for (int i = 0; i < m_; i++) cj[i] += ap[i] * bpj;
            }
        }
    }

  private:
    int m_, n_, k_, lda_, ldb_, ldc_;
};

#endif /* LFFN_STANDIN_LIBXSMM_H_ */
