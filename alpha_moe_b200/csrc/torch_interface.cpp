// torch operator boundary: alpha_moe::fused_moe_w8a8_up_down on the CUDA dispatch key.
//
// Drop-in for csrc/torch_interface.cpp:37-127 of the reference: identical schema string, identical
// knob checks (:62-64) and contiguity checks (:66-76); on top of those it checks what the reference
// leaves unchecked (dtypes, device, shapes of w2 / scales / out).  The stream is fetched after the
// device guard is installed.  All work happens in the C ABI library; this file holds no CUDA code.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/library.h>

#include "../../include/alpha_moe_b200.h"

namespace {

void fused_moe_w8a8_up_down(const torch::Tensor& x, const torch::Tensor& x_scale, const torch::Tensor& w,
                            const torch::Tensor& w_scale, const torch::Tensor& w2, const torch::Tensor& w2_scale,
                            const torch::Tensor& sorted_token_ids, const torch::Tensor& expert_ids,
                            const torch::Tensor& num_tokens_post_padded, const torch::Tensor& topk_weights,
                            torch::Tensor& out, int64_t top_k, int64_t block_m, int64_t block_n, int64_t warp_n,
                            int64_t stages, double scaling_factor) {
    const at::cuda::OptionalCUDAGuard device_guard(device_of(x));
    const cudaStream_t stream = at::cuda::getCurrentCUDAStream();

    TORCH_CHECK(x.dim() == 2 && w.dim() == 3 && w2.dim() == 3, "x must be [M,K], w [E,N,K], w2 [E,K,N/2]");
    TORCH_CHECK(x.size(0), "x must have at least one row");
    TORCH_CHECK(x.size(1) == w.size(2), "x.size(1) must equal w.size(2)");
    TORCH_CHECK(x.size(1) % 128 == 0, "K dimension must be a multiple of 128");
    TORCH_CHECK((block_n == 64 && warp_n == 4) || (block_n == 32 && warp_n == 8),
                "(block_n, warp_n) must be (64,4) or (32,8)");
    TORCH_CHECK(stages > 0 && stages < 6, "stages must be in 1..5");
    TORCH_CHECK(block_m > 0 && block_m <= 128 && block_m % 8 == 0, "block_m must be a multiple of 8 in 8..128");

    TORCH_CHECK(x.is_contiguous() && w.is_contiguous() && w2.is_contiguous(), "x, w, w2 must be contiguous");
    TORCH_CHECK(x_scale.is_contiguous() && w_scale.is_contiguous() && w2_scale.is_contiguous(),
                "scales must be contiguous");
    TORCH_CHECK(sorted_token_ids.is_contiguous() && expert_ids.is_contiguous() && topk_weights.is_contiguous() &&
                    num_tokens_post_padded.is_contiguous() && out.is_contiguous(),
                "index tensors, topk_weights and out must be contiguous");

    const int64_t M = x.size(0), K = x.size(1), E = w.size(0), N = w.size(1);
    TORCH_CHECK(N % 256 == 0, "N (2 x intermediate size) must be a multiple of 256");
    TORCH_CHECK(w2.size(0) == E && w2.size(1) == K && w2.size(2) == N / 2, "w2 must be [E, K, N/2]");
    TORCH_CHECK(x.element_size() == 1 && w.element_size() == 1 && w2.element_size() == 1,
                "x, w, w2 must be 8-bit (float8_e4m3fn)");
    TORCH_CHECK(x.scalar_type() == w.scalar_type() && w.scalar_type() == w2.scalar_type(),
                "x, w, w2 must share one dtype");
    TORCH_CHECK(x_scale.scalar_type() == at::kFloat && w_scale.scalar_type() == at::kFloat &&
                    w2_scale.scalar_type() == at::kFloat && topk_weights.scalar_type() == at::kFloat,
                "scales and topk_weights must be float32");
    TORCH_CHECK(sorted_token_ids.scalar_type() == at::kInt && expert_ids.scalar_type() == at::kInt &&
                    num_tokens_post_padded.scalar_type() == at::kInt,
                "sorted_token_ids, expert_ids, num_tokens_post_padded must be int32");
    TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == M && out.size(1) == K,
                "out must be bfloat16 [M, K]");
    TORCH_CHECK(x_scale.numel() == M * (K / 128), "x_scale must be [M, K/128]");
    TORCH_CHECK(w_scale.numel() == E * (N / 128) * (K / 128), "w_scale must be [E, N/128, K/128]");
    TORCH_CHECK(w2_scale.numel() == E * (K / 128) * (N / 256), "w2_scale must be [E, K/128, N/256]");
    TORCH_CHECK(topk_weights.numel() == M * top_k, "topk_weights must be [M, top_k]");
    TORCH_CHECK(expert_ids.numel() * block_m >= sorted_token_ids.numel(),
                "expert_ids must hold one entry per block_m sorted slots");
    TORCH_CHECK(num_tokens_post_padded.numel() >= 1, "num_tokens_post_padded must hold one element");
    for (const torch::Tensor* t : {&x_scale, &w, &w_scale, &w2, &w2_scale, &sorted_token_ids, &expert_ids,
                                   &num_tokens_post_padded, &topk_weights, static_cast<const torch::Tensor*>(&out)})
        TORCH_CHECK(t->is_cuda() && t->device() == x.device(), "all tensors must live on x's CUDA device");

    const int rc = alpha_moe_b200_fused_moe_w8a8_up_down(
        x.data_ptr(), static_cast<const float*>(x_scale.data_ptr()), w.data_ptr(),
        static_cast<const float*>(w_scale.data_ptr()), w2.data_ptr(), static_cast<const float*>(w2_scale.data_ptr()),
        out.data_ptr(), static_cast<const int32_t*>(sorted_token_ids.data_ptr()),
        static_cast<const int32_t*>(expert_ids.data_ptr()),
        static_cast<const int32_t*>(num_tokens_post_padded.data_ptr()),
        static_cast<const float*>(topk_weights.data_ptr()), static_cast<int>(top_k), static_cast<int>(M),
        static_cast<int>(K), static_cast<int>(N), static_cast<int>(E), static_cast<int>(sorted_token_ids.numel()),
        static_cast<int>(block_m), static_cast<int>(block_n), static_cast<int>(warp_n), static_cast<int>(stages),
        static_cast<float>(scaling_factor), stream);
    TORCH_CHECK(rc == ALPHA_MOE_OK, "alpha_moe_b200: ", alpha_moe_b200_last_error());
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(alpha_moe, m) {
    m.def(
        "fused_moe_w8a8_up_down("
        "Tensor x, "
        "Tensor x_scale, "
        "Tensor w, "
        "Tensor w_scale, "
        "Tensor w2, "
        "Tensor w2_scale, "
        "Tensor sorted_token_ids, "
        "Tensor expert_ids, "
        "Tensor num_tokens_post_padded, "
        "Tensor topk_weights, "
        "Tensor(a!) out, "
        "int top_k, "
        "int block_m, "
        "int block_n, "
        "int warp_n, "
        "int stages, "
        "float scaling_factor"
        ") -> ()");
    m.impl("fused_moe_w8a8_up_down", torch::kCUDA, &fused_moe_w8a8_up_down);
}
