// Host API of the tcgen05 bf16 GEMM family.
#pragma once
#include <cuda_runtime.h>

namespace z2h {

// Epilogue selector.
enum GemmEpilogue : int {
  kEpiNone = 0,        // C = acc (+ bias)
  kEpiResidual = 1,    // C = acc (+ bias) + residual
  kEpiGelu = 2,        // aux_out = acc (+ bias);  C = gelu_tanh(aux_out)
  kEpiGeluGrad = 3,    // C = acc * gelu_tanh'(aux_in)
  kEpiAtomicAdd = 4,   // C(fp32) += acc with red.global.add (split-K capable)
  kEpiAccumulate = 5,  // C(fp32) += acc with plain read-modify-write (deterministic)
  // The pair a training step uses for the MLP: the forward GEMM stores the DERIVATIVE of the
  // activation instead of the pre-activation (the backward needs nothing else of it, and both share
  // one tanh), so the backward epilogue is one load and one multiply instead of a second GELU'.
  kEpiGeluSaveGrad = 6,  // x = acc (+ bias); aux_out = gelu_tanh'(x); C = gelu_tanh(x)
  kEpiMulAux = 7,        // C = acc * aux_in
  // Split-K without atomics: K-slice s of a tile is stored (not added) at C + s * slice_stride, fp32;
  // gemm_fold_slices then adds the slices to their destination in slice order. Together they are the
  // bitwise reproducible form of a split-K weight gradient.
  kEpiSliceStore = 8,
};

// C[M,N] = A * B^T in the logical sense: A is M x K, B is N x K.
// a_mn == 0: A is stored row-major [M, K] with pitch lda   (K-major)
// a_mn == 1: A is stored row-major [K, M] with pitch lda   (MN-major, i.e. A^T in memory)
// b_mn == 0: B is stored row-major [N, K] with pitch ldb   (K-major)
// b_mn == 1: B is stored row-major [K, N] with pitch ldb   (MN-major)
// All pitches are in elements and must be multiples of 8; base pointers 16-byte aligned.
struct GemmArgs {
  const void* A; int a_mn; long long lda;
  const void* B; int b_mn; long long ldb;
  void* C; long long ldc; int out_fp32;
  int M, N, K;
  int epi;
  int split_k;            // > 1: K cut into slices; <= 0 with kEpiAtomicAdd: stream-K (one run of k-blocks per SM)
  const void* bias;       // bf16 [N] or null
  const void* residual;   // bf16 [M, ldr]
  long long ldr;
  void* aux_out;          // bf16 [M, ldaux]
  const void* aux_in;     // bf16 [M, ldaux]
  long long ldaux;
  int* status;            // device status word (0 == ok), may be null
  // fp32 [N] or null: the column sums of C (as stored, i.e. rounded to bf16) are ADDED to it, which
  // makes the bias gradient of the layer below a by-product of the GEMM that produces that layer's
  // output gradient. Needs a bf16 output, split_k == 1, M % 32 == 0 and N % 32 == 0.
  void* colsum;
  long long slice_stride;  // kEpiSliceStore: elements between the outputs of consecutive K-slices
  int max_ctas;           // 0 = one CTA per SM
};

// Returns 0 on success, 1 bad argument, 2 tensor-map encoding failed, 3 launch failed.
// Validates the arguments and picks the kernel (see gemm_set_algo).
int gemm_bf16(const GemmArgs& args, cudaStream_t stream);

// The CTA-pair kernel (256 x 256 tiles, tcgen05.mma.cta_group::2); arguments already validated.
int gemm_bf16_pair(const GemmArgs& args, cudaStream_t stream);

// 0: always the one-CTA kernel (128 x 256 tiles); 1: the CTA-pair kernel whenever M >= 256;
// 2 (default): CTA pairs when the problem has at least one 256 x 256 tile per pair of SMs.
void gemm_set_algo(int algo);
// dst[i] += slices[0][i] + slices[1][i] + ... (in that order), n elements per slice, n % 4 == 0.
int gemm_fold_slices(const float* slices, int num_slices, long long n, float* dst, cudaStream_t stream);
// Stream-K with fix-up in the CTA-pair kernel (balanced k-block runs for tile counts that leave a
// ragged last wave; see gemm_tcgen05_2cta.cu): 0 off (default: it measured slower), 1 on (also
// Z2H_GEMM_FIXUP=1).
void gemm_set_fixup(int on);
int gemm_get_algo();

}  // namespace z2h
