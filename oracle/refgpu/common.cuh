// TEST INFRASTRUCTURE.  Stand-in for the header of this name that the reference's src/kernels.cu includes from its
// un-vendored dependency (ggml-cuda of llama.cpp): only the declarations kernels.cu needs in order to compile - the
// published q8_1 block format, the GGUF type numbers and the block sizes of the formats it names.  Written for this
// build; nothing here comes from that dependency's sources.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>
#define QK8_1 32
struct block_q8_1 {      // the published q8_1 block: f16 d, f16 sum, 32 int8
    half2 ds;
    int8_t qs[QK8_1];
};
enum ggml_type { GGML_TYPE_Q4_0 = 2, GGML_TYPE_Q5_1 = 7, GGML_TYPE_Q8_0 = 8, GGML_TYPE_Q4_K = 12, GGML_TYPE_Q5_K = 13, GGML_TYPE_Q6_K = 14, GGML_TYPE_IQ4_NL = 20 };
template <ggml_type t> struct ggml_cuda_type_traits;
template <> struct ggml_cuda_type_traits<GGML_TYPE_Q4_0> { static constexpr int qk = 32, qr = 2, qi = 4; };
template <> struct ggml_cuda_type_traits<GGML_TYPE_Q5_1> { static constexpr int qk = 32, qr = 2, qi = 4; };
template <> struct ggml_cuda_type_traits<GGML_TYPE_Q8_0> { static constexpr int qk = 32, qr = 1, qi = 8; };
template <> struct ggml_cuda_type_traits<GGML_TYPE_Q4_K> { static constexpr int qk = 256, qr = 2, qi = 32; };
template <> struct ggml_cuda_type_traits<GGML_TYPE_Q5_K> { static constexpr int qk = 256, qr = 2, qi = 32; };
template <> struct ggml_cuda_type_traits<GGML_TYPE_Q6_K> { static constexpr int qk = 256, qr = 2, qi = 32; };
template <> struct ggml_cuda_type_traits<GGML_TYPE_IQ4_NL> { static constexpr int qk = 32, qr = 2, qi = 4; };
