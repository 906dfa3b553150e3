// TEST INFRASTRUCTURE.  Stand-in for the second header src/kernels.cu includes from its un-vendored dependency.  That
// header holds the dependency's quantised dot products; they are NOT restated here: the functions below return 0 and
// exist only so that the reference's templates instantiate.  The kernels that call them (mmvq, the generic expert
// kernels and the down projection) are compiled but never run by the tests; the kernels the tests do run (the router,
// the Q4_K gate|up, the split-Q8_0 dense kernel, the DeltaNet core, the attention scan, argmax and the top-64) carry
// their whole arithmetic in the reference's own tree.  The VDR values only shape those unused instantiations.
#pragma once
#define VDR_Q8_0_Q8_1_MMVQ 2
#define VDR_Q4_K_Q8_1_MMVQ 2
#define VDR_Q5_K_Q8_1_MMVQ 2
#define VDR_Q5_1_Q8_1_MMVQ 2
#define VDR_Q4_0_Q8_1_MMVQ 2
#define VDR_Q6_K_Q8_1_MMVQ 1
#define VDR_IQ4_NL_Q8_1_MMVQ 2
#define FNX_REF_NO_DOT(name) static __device__ __forceinline__ float name(const void*, const block_q8_1*, const int&, const int&) { return 0.f; }
FNX_REF_NO_DOT(vec_dot_q8_0_q8_1) FNX_REF_NO_DOT(vec_dot_q4_K_q8_1) FNX_REF_NO_DOT(vec_dot_q5_K_q8_1) FNX_REF_NO_DOT(vec_dot_q5_1_q8_1)
FNX_REF_NO_DOT(vec_dot_q4_0_q8_1) FNX_REF_NO_DOT(vec_dot_q6_K_q8_1) FNX_REF_NO_DOT(vec_dot_iq4_nl_q8_1)
