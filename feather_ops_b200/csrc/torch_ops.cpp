// Thin torch extension over the C ABI: registers the `torch.ops.feather_ops.*` operators: four with the
// schemas of the reference (csrc/hip_kernel.cu:825-846, csrc/hip_kernel_int8.cu:564-586 and :972-980,
// csrc/hip_conv2d_3x3.cu:672-692) and `scaled_mm_splitk` (the skinny-M launcher over caller scratch, no
// counterpart in the reference). It validates tensors with the reference's messages, takes the current
// CUDA stream of the input's device and forwards raw pointers to libfeather_ops_b200.so. Built against
// torch's stable ABI, so it does not depend on libtorch_python. Nothing here computes or allocates.
#include <Python.h>

#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/headeronly/core/ScalarType.h>
#include <torch/headeronly/util/Exception.h>

#include <cstdint>
#include <optional>

#include "feather_ops_b200.h"

namespace {

using torch::stable::Tensor;
using ScalarType = torch::headeronly::ScalarType;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 0xFu) == 0u; }

feather_stream_t current_stream(int32_t device_index) {
    void* raw = nullptr;
    TORCH_ERROR_CODE_CHECK(aoti_torch_get_current_cuda_stream(device_index, &raw));
    return reinterpret_cast<feather_stream_t>(raw);
}

bool is_half_or_bf16(ScalarType t) { return t == ScalarType::Half || t == ScalarType::BFloat16; }

void scaled_mm(const Tensor& a, const Tensor& b_prepacked, const std::optional<Tensor>& scale, const std::optional<Tensor>& bias, Tensor& c,
               int64_t block_warps_m, int64_t block_warps_n, int64_t unroll_k, int64_t repeat_m, int64_t repeat_n, bool prefetch) {
    STD_TORCH_CHECK(a.is_cuda(), "a must be a CUDA tensor");
    STD_TORCH_CHECK(b_prepacked.is_cuda(), "b_prepacked must be a CUDA tensor");
    STD_TORCH_CHECK(c.is_cuda(), "c must be a CUDA tensor");
    const auto device = a.get_device_index();
    STD_TORCH_CHECK(b_prepacked.get_device_index() == device, "b_prepacked must be on the same device as a");
    STD_TORCH_CHECK(c.get_device_index() == device, "c must be on the same device as a");

    STD_TORCH_CHECK(is_half_or_bf16(a.scalar_type()), "a must be float16 or bfloat16");
    STD_TORCH_CHECK(is_half_or_bf16(c.scalar_type()), "c must be float16 or bfloat16");
    const auto b_type = b_prepacked.scalar_type();
    STD_TORCH_CHECK(b_type == ScalarType::Float8_e4m3fn || b_type == ScalarType::Float8_e5m2, "b_prepacked must be float8_e4m3fn or float8_e5m2");

    STD_TORCH_CHECK(a.dim() == 2, "a must be 2D");
    STD_TORCH_CHECK(b_prepacked.dim() == 3, "b_prepacked must be 3D (K/16, N, 16)");
    STD_TORCH_CHECK(c.dim() == 2, "c must be 2D");
    const int64_t M = a.size(0);
    const int64_t K = a.size(1);
    const int64_t N = b_prepacked.size(1);
    STD_TORCH_CHECK(K % 16 == 0, "K must be divisible by 16");
    STD_TORCH_CHECK(N % 16 == 0, "N must be divisible by 16");
    STD_TORCH_CHECK(b_prepacked.size(0) >= K / 16, "b_prepacked.shape[0] must be at least K/16 (", K / 16, ")");
    STD_TORCH_CHECK(b_prepacked.size(0) % 8 == 0, "b_prepacked.shape[0] must be a multiple of 8 (K padded to 128)");
    STD_TORCH_CHECK(b_prepacked.size(2) == 16, "b_prepacked.shape[2] must be 16");
    STD_TORCH_CHECK(c.size(0) == M, "c.shape[0] must equal M");
    STD_TORCH_CHECK(c.size(1) == N, "c.shape[1] must equal N");

    STD_TORCH_CHECK(a.stride(0) == K, "a.stride(0) must equal K (", K, ")");
    STD_TORCH_CHECK(a.stride(1) == 1, "a.stride(1) must be 1");
    STD_TORCH_CHECK(b_prepacked.stride(0) == N * 16, "b_prepacked.stride(0) must equal N*16 (", N * 16, ")");
    STD_TORCH_CHECK(b_prepacked.stride(1) == 16, "b_prepacked.stride(1) must be 16");
    STD_TORCH_CHECK(b_prepacked.stride(2) == 1, "b_prepacked.stride(2) must be 1");
    STD_TORCH_CHECK(c.stride(0) == N, "c.stride(0) must equal N (", N, ")");
    STD_TORCH_CHECK(c.stride(1) == 1, "c.stride(1) must be 1");

    if (scale.has_value()) {
        STD_TORCH_CHECK(scale->is_cuda(), "scale must be a CUDA tensor");
        STD_TORCH_CHECK(scale->get_device_index() == device, "scale must be on the same device as a");
        STD_TORCH_CHECK(scale->scalar_type() == ScalarType::Float, "scale must be float32");
        STD_TORCH_CHECK(scale->numel() == 1, "scale must have one element");
    }
    if (bias.has_value()) {
        STD_TORCH_CHECK(bias->is_cuda(), "bias must be a CUDA tensor");
        STD_TORCH_CHECK(bias->get_device_index() == device, "bias must be on the same device as a");
        STD_TORCH_CHECK(bias->scalar_type() == c.scalar_type(), "bias must have the same dtype as c");
        STD_TORCH_CHECK(bias->numel() == N, "bias must have N elements");
        STD_TORCH_CHECK(bias->is_contiguous(), "bias must be contiguous");
    }

    torch::stable::accelerator::DeviceGuard guard(device);
    const feather_stream_t stream = current_stream(device);

    STD_TORCH_CHECK(aligned16(a.const_data_ptr()), "a data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(b_prepacked.const_data_ptr()), "b_prepacked data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(c.mutable_data_ptr()), "c data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(32 * block_warps_m * block_warps_n <= 1024, "Block size exceeds the thread-per-block limit");

    const bool launched = launch_scaled_mm(
        static_cast<const uint16_t*>(a.const_data_ptr()), static_cast<const uint8_t*>(b_prepacked.const_data_ptr()),
        scale.has_value() ? static_cast<const float*>(scale->const_data_ptr()) : nullptr,
        bias.has_value() ? static_cast<const uint16_t*>(bias->const_data_ptr()) : nullptr, static_cast<uint16_t*>(c.mutable_data_ptr()), M, N, K,
        scale.has_value() ? 1 : 0, bias.has_value() ? 1 : 0, b_type == ScalarType::Float8_e5m2, a.scalar_type() == ScalarType::BFloat16,
        c.scalar_type() == ScalarType::BFloat16, static_cast<int>(block_warps_m), static_cast<int>(block_warps_n), static_cast<int>(unroll_k),
        static_cast<int>(repeat_m), static_cast<int>(repeat_n), prefetch, stream);
    STD_TORCH_CHECK(launched, "Unsupported config");
}

// Split-K scaled_mm. `block_n` 64: the skinny kernel (M <= 128); 128 or 256: the one-CTA kernel walking (tile, K split)
// items, any M. Same tensor contract as `scaled_mm`, plus caller-provided scratch: `partials` (float32, at least
// feather_scaled_mm_splitk_partial_floats elements) and `counters` (int32 zeros, one per tile of 128 x block_n; ceil(N / 64)
// for the skinny kernel). The Python wrapper allocates both with torch, so they are stream ordered.
void scaled_mm_splitk(const Tensor& a, const Tensor& b_prepacked, const std::optional<Tensor>& scale, const std::optional<Tensor>& bias, Tensor& c,
                      Tensor& partials, Tensor& counters, int64_t splits, int64_t block_n) {
    STD_TORCH_CHECK(a.is_cuda() && b_prepacked.is_cuda() && c.is_cuda() && partials.is_cuda() && counters.is_cuda(), "tensors must be CUDA tensors");
    const auto device = a.get_device_index();
    STD_TORCH_CHECK(b_prepacked.get_device_index() == device && c.get_device_index() == device && partials.get_device_index() == device &&
                        counters.get_device_index() == device,
                    "all tensors must be on the same device as a");
    STD_TORCH_CHECK(is_half_or_bf16(a.scalar_type()), "a must be float16 or bfloat16");
    STD_TORCH_CHECK(is_half_or_bf16(c.scalar_type()), "c must be float16 or bfloat16");
    const auto b_type = b_prepacked.scalar_type();
    STD_TORCH_CHECK(b_type == ScalarType::Float8_e4m3fn || b_type == ScalarType::Float8_e5m2, "b_prepacked must be float8_e4m3fn or float8_e5m2");
    STD_TORCH_CHECK(a.dim() == 2 && c.dim() == 2, "a and c must be 2D");
    STD_TORCH_CHECK(b_prepacked.dim() == 3 && b_prepacked.size(2) == 16, "b_prepacked must be 3D (K/16, N, 16)");
    const int64_t M = a.size(0);
    const int64_t K = a.size(1);
    const int64_t N = b_prepacked.size(1);
    STD_TORCH_CHECK(block_n == 64 || block_n == 128 || block_n == 256, "block_n must be 64, 128 or 256");
    STD_TORCH_CHECK(block_n != 64 || M <= 128, "the 64-wide split-K path is for M <= 128");
    STD_TORCH_CHECK(K % 16 == 0, "K must be divisible by 16");
    STD_TORCH_CHECK(N % 16 == 0, "N must be divisible by 16");
    STD_TORCH_CHECK(b_prepacked.size(0) >= K / 16 && b_prepacked.size(0) % 8 == 0, "b_prepacked.shape[0] must cover K padded to 128");
    STD_TORCH_CHECK(c.size(0) == M && c.size(1) == N, "c must be [M, N]");
    STD_TORCH_CHECK(a.is_contiguous() && b_prepacked.is_contiguous() && c.is_contiguous(), "a, b_prepacked and c must be contiguous");
    STD_TORCH_CHECK(partials.scalar_type() == ScalarType::Float && partials.is_contiguous(), "partials must be contiguous float32");
    STD_TORCH_CHECK(counters.scalar_type() == ScalarType::Int && counters.is_contiguous(), "counters must be contiguous int32");
    const int64_t scratch = block_n == 64 ? feather_scaled_mm_splitk_partial_floats(M, N, K, static_cast<int>(splits))
                                          : feather_scaled_mm_splitk_wide_partial_floats(M, N, K, static_cast<int>(block_n), static_cast<int>(splits));
    STD_TORCH_CHECK(partials.numel() >= scratch, "partials is too small");
    const int64_t tickets = block_n == 64 ? (N + 63) / 64 : feather_scaled_mm_splitk_wide_counters(M, N, static_cast<int>(block_n));
    STD_TORCH_CHECK(counters.numel() >= tickets, "counters must have one element per tile");
    if (scale.has_value()) {
        STD_TORCH_CHECK(scale->is_cuda() && scale->scalar_type() == ScalarType::Float && scale->numel() == 1, "scale must be one float32 on the device");
        STD_TORCH_CHECK(scale->get_device_index() == device, "scale must be on the same device as a");
    }
    if (bias.has_value()) {
        STD_TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == c.scalar_type() && bias->numel() == N && bias->is_contiguous(),
                        "bias must be N contiguous elements of c's dtype");
        STD_TORCH_CHECK(bias->get_device_index() == device, "bias must be on the same device as a");
    }
    STD_TORCH_CHECK(aligned16(a.const_data_ptr()) && aligned16(b_prepacked.const_data_ptr()) && aligned16(c.mutable_data_ptr()) &&
                        aligned16(partials.mutable_data_ptr()),
                    "data pointers must be 16-byte aligned");
    torch::stable::accelerator::DeviceGuard guard(device);
    const feather_stream_t stream = current_stream(device);
    const uint16_t* const a_ptr = static_cast<const uint16_t*>(a.const_data_ptr());
    const uint8_t* const b_ptr = static_cast<const uint8_t*>(b_prepacked.const_data_ptr());
    const float* const scale_ptr = scale.has_value() ? static_cast<const float*>(scale->const_data_ptr()) : nullptr;
    const uint16_t* const bias_ptr = bias.has_value() ? static_cast<const uint16_t*>(bias->const_data_ptr()) : nullptr;
    uint16_t* const c_ptr = static_cast<uint16_t*>(c.mutable_data_ptr());
    float* const partials_ptr = static_cast<float*>(partials.mutable_data_ptr());
    uint32_t* const counters_ptr = static_cast<uint32_t*>(counters.mutable_data_ptr());
    const bool e5m2 = b_type == ScalarType::Float8_e5m2;
    const bool a_bf16 = a.scalar_type() == ScalarType::BFloat16;
    const bool c_bf16 = c.scalar_type() == ScalarType::BFloat16;
    const bool launched =
        block_n == 64 ? launch_scaled_mm_splitk(a_ptr, b_ptr, scale_ptr, bias_ptr, c_ptr, M, N, K, scale.has_value() ? 1 : 0, bias.has_value() ? 1 : 0,
                                                e5m2, a_bf16, c_bf16, static_cast<int>(splits), partials_ptr, counters_ptr, stream)
                      : launch_scaled_mm_splitk_wide(a_ptr, b_ptr, scale_ptr, bias_ptr, c_ptr, M, N, K, scale.has_value() ? 1 : 0,
                                                     bias.has_value() ? 1 : 0, e5m2, a_bf16, c_bf16, static_cast<int>(block_n),
                                                     static_cast<int>(splits), partials_ptr, counters_ptr, stream);
    STD_TORCH_CHECK(launched, "scaled_mm_splitk: unsupported problem");
}

// out[r, g * width : (g + 1) * width] = slabs[g, r, :]: the row-major matrix from the [world, rows, width] all-gather of column slabs.
void interleave_slabs(const Tensor& slabs, Tensor& out) {
    STD_TORCH_CHECK(slabs.is_cuda() && out.is_cuda() && slabs.get_device_index() == out.get_device_index(), "slabs and out must be on one CUDA device");
    STD_TORCH_CHECK(slabs.dim() == 3 && out.dim() == 2, "slabs must be [world, rows, width], out [rows, world * width]");
    STD_TORCH_CHECK(slabs.scalar_type() == out.scalar_type(), "slabs and out must have the same dtype");
    STD_TORCH_CHECK(is_half_or_bf16(out.scalar_type()), "slabs must be float16 or bfloat16");
    const int64_t world = slabs.size(0), rows = slabs.size(1), width = slabs.size(2);
    STD_TORCH_CHECK(out.size(0) == rows && out.size(1) == world * width, "out must be [rows, world * width]");
    STD_TORCH_CHECK(slabs.is_contiguous() && out.is_contiguous(), "slabs and out must be contiguous");
    STD_TORCH_CHECK(width % 8 == 0, "the slab width must be a multiple of 8 elements");
    STD_TORCH_CHECK(aligned16(slabs.const_data_ptr()) && aligned16(out.mutable_data_ptr()), "data pointers must be 16-byte aligned");
    const auto device = slabs.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);
    STD_TORCH_CHECK(launch_interleave_slabs(slabs.const_data_ptr(), out.mutable_data_ptr(), world, rows, width * 2, current_stream(device)), "interleave_slabs launch failed");
}

void int8_scaled_mm(const Tensor& a, const Tensor& b_prepacked, const Tensor& a_scale, const std::optional<Tensor>& b_scale,
                    const std::optional<Tensor>& bias, Tensor& c, bool transposed_b, int64_t block_warps_m, int64_t block_warps_n,
                    int64_t unroll_k, int64_t repeat_m, int64_t repeat_n) {
    STD_TORCH_CHECK(a.is_cuda(), "a must be a CUDA tensor");
    STD_TORCH_CHECK(b_prepacked.is_cuda(), "b_prepacked must be a CUDA tensor");
    STD_TORCH_CHECK(c.is_cuda(), "c must be a CUDA tensor");
    const auto device = a.get_device_index();
    STD_TORCH_CHECK(b_prepacked.get_device_index() == device, "b_prepacked must be on the same device as a");
    STD_TORCH_CHECK(c.get_device_index() == device, "c must be on the same device as a");
    STD_TORCH_CHECK(a.scalar_type() == ScalarType::Char, "a must be int8");
    STD_TORCH_CHECK(b_prepacked.scalar_type() == ScalarType::Char, "b_prepacked must be int8");
    STD_TORCH_CHECK(is_half_or_bf16(c.scalar_type()), "c must be float16 or bfloat16");
    STD_TORCH_CHECK(a.dim() == 2, "a must be 2D");
    STD_TORCH_CHECK(c.dim() == 2, "c must be 2D");

    const int64_t M = a.size(0);
    const int64_t K_contract = a.size(1);
    const int64_t N_out = c.size(1);
    const int64_t weight_in = transposed_b ? N_out : K_contract;
    const int64_t weight_out = transposed_b ? K_contract : N_out;
    STD_TORCH_CHECK(b_prepacked.numel() == weight_in * weight_out, "b_prepacked must hold weight_in * weight_out bytes");
    STD_TORCH_CHECK(weight_in % 4 == 0 && weight_out % 4 == 0, "the weight axes must be multiples of 4");
    STD_TORCH_CHECK(K_contract % 16 == 0, "the contraction axis must be a multiple of 16");
    STD_TORCH_CHECK(c.size(0) == M, "c.shape[0] must equal M");
    STD_TORCH_CHECK(a.stride(0) == K_contract && a.stride(1) == 1, "a must be contiguous");
    STD_TORCH_CHECK(c.stride(0) == N_out && c.stride(1) == 1, "c must be contiguous");
    STD_TORCH_CHECK(b_prepacked.is_contiguous(), "b_prepacked must be contiguous");
    STD_TORCH_CHECK(a_scale.is_cuda() && a_scale.scalar_type() == ScalarType::Float, "a_scale must be float32");
    STD_TORCH_CHECK(a_scale.get_device_index() == device, "a_scale must be on the same device as a");
    STD_TORCH_CHECK(a_scale.numel() == M, "a_scale must have M elements");
    STD_TORCH_CHECK(a_scale.is_contiguous(), "a_scale must be contiguous");
    if (b_scale.has_value()) {
        STD_TORCH_CHECK(b_scale->is_cuda() && b_scale->scalar_type() == ScalarType::Float, "b_scale must be float32");
        STD_TORCH_CHECK(b_scale->get_device_index() == device, "b_scale must be on the same device as a");
        STD_TORCH_CHECK(b_scale->numel() == N_out, "b_scale must have N elements");
        STD_TORCH_CHECK(b_scale->is_contiguous(), "b_scale must be contiguous");
    }
    if (bias.has_value()) {
        STD_TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == c.scalar_type(), "bias must have the same dtype as c");
        STD_TORCH_CHECK(bias->get_device_index() == device, "bias must be on the same device as a");
        STD_TORCH_CHECK(bias->numel() == N_out, "bias must have N elements");
        STD_TORCH_CHECK(bias->is_contiguous(), "bias must be contiguous");
    }
    STD_TORCH_CHECK(aligned16(a.const_data_ptr()), "a data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(b_prepacked.const_data_ptr()), "b_prepacked data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(c.mutable_data_ptr()), "c data pointer must be 16-byte aligned");

    torch::stable::accelerator::DeviceGuard guard(device);
    const feather_stream_t stream = current_stream(device);

    // Micro-tile (k4, n4) sits at index k4 * (weight_out / 4) + n4: the contraction axis is the outer one
    // for the forward and the inner one for the backward.
    const int64_t inner = weight_out / 4;
    const int64_t stride_kc = transposed_b ? 1 : inner;
    const int64_t stride_out = transposed_b ? inner : 1;
    const bool launched = launch_int8_scaled_mm(
        static_cast<const int8_t*>(a.const_data_ptr()), static_cast<const uint8_t*>(b_prepacked.const_data_ptr()),
        static_cast<const float*>(a_scale.const_data_ptr()), b_scale.has_value() ? static_cast<const float*>(b_scale->const_data_ptr()) : nullptr,
        bias.has_value() ? static_cast<const uint16_t*>(bias->const_data_ptr()) : nullptr, static_cast<uint16_t*>(c.mutable_data_ptr()), M, N_out,
        K_contract, stride_kc, stride_out, transposed_b, static_cast<int>(block_warps_m), static_cast<int>(block_warps_n),
        static_cast<int>(unroll_k), static_cast<int>(repeat_m), static_cast<int>(repeat_n), c.scalar_type() == ScalarType::Half ? 0 : 1, stream);
    STD_TORCH_CHECK(launched, "Unsupported config");
}

// The int8 GEMM over the released row-major `[N, K]` weight (no prepack). Not in the reference's schema list: it backs the
// `weight_packed=False` calls of the Python API.
void int8_scaled_mm_plain(const Tensor& a, const Tensor& weight, const Tensor& a_scale, const std::optional<Tensor>& b_scale,
                          const std::optional<Tensor>& bias, Tensor& c, bool transposed_b) {
    STD_TORCH_CHECK(a.is_cuda() && weight.is_cuda() && c.is_cuda(), "tensors must be CUDA tensors");
    const auto device = a.get_device_index();
    STD_TORCH_CHECK(weight.get_device_index() == device && c.get_device_index() == device, "tensors must be on the same device");
    STD_TORCH_CHECK(a.scalar_type() == ScalarType::Char && weight.scalar_type() == ScalarType::Char, "a and weight must be int8");
    STD_TORCH_CHECK(is_half_or_bf16(c.scalar_type()), "c must be float16 or bfloat16");
    STD_TORCH_CHECK(a.dim() == 2 && weight.dim() == 2 && c.dim() == 2, "a, weight and c must be 2D");
    const int64_t M = a.size(0);
    const int64_t N = weight.size(0);
    const int64_t K = weight.size(1);
    STD_TORCH_CHECK(a.size(1) == (transposed_b ? N : K), "a's row length must equal the weight axis that is contracted");
    STD_TORCH_CHECK(c.size(0) == M && c.size(1) == (transposed_b ? K : N), "c has the wrong shape");
    STD_TORCH_CHECK(K % 16 == 0 && N % (transposed_b ? 16 : 4) == 0, "the weight axes must be multiples of 16 (forward: out_features of 4)");
    STD_TORCH_CHECK(a.is_contiguous() && weight.is_contiguous() && c.is_contiguous(), "a, weight and c must be contiguous");
    STD_TORCH_CHECK(a_scale.is_cuda() && a_scale.scalar_type() == ScalarType::Float && a_scale.get_device_index() == device, "a_scale must be float32 on a's device");
    STD_TORCH_CHECK(a_scale.numel() == M && a_scale.is_contiguous(), "a_scale must have M contiguous elements");
    STD_TORCH_CHECK(!transposed_b || (!b_scale.has_value() && !bias.has_value()), "transposed_b takes neither b_scale nor bias");
    if (b_scale.has_value()) {
        STD_TORCH_CHECK(b_scale->is_cuda() && b_scale->scalar_type() == ScalarType::Float && b_scale->get_device_index() == device, "b_scale must be float32 on a's device");
        STD_TORCH_CHECK(b_scale->numel() == N && b_scale->is_contiguous(), "b_scale must have N contiguous elements");
    }
    if (bias.has_value()) {
        STD_TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == c.scalar_type() && bias->get_device_index() == device, "bias must have c's dtype and device");
        STD_TORCH_CHECK(bias->numel() == N && bias->is_contiguous(), "bias must have N contiguous elements");
    }
    STD_TORCH_CHECK(aligned16(a.const_data_ptr()) && aligned16(weight.const_data_ptr()) && aligned16(c.mutable_data_ptr()), "data pointers must be 16-byte aligned");
    torch::stable::accelerator::DeviceGuard guard(device);
    const bool launched = launch_int8_scaled_mm_plain(
        static_cast<const int8_t*>(a.const_data_ptr()), static_cast<const int8_t*>(weight.const_data_ptr()), static_cast<const float*>(a_scale.const_data_ptr()),
        b_scale.has_value() ? static_cast<const float*>(b_scale->const_data_ptr()) : nullptr,
        bias.has_value() ? static_cast<const uint16_t*>(bias->const_data_ptr()) : nullptr, static_cast<uint16_t*>(c.mutable_data_ptr()), M, N, K, transposed_b,
        c.scalar_type() == ScalarType::Half ? 0 : 1, current_stream(device));
    STD_TORCH_CHECK(launched, "int8_scaled_mm_plain launch failed");
}

void convrot_quantize(const Tensor& x, const std::optional<Tensor>& col_scale, Tensor& q, Tensor& row_scale, bool rotate) {
    STD_TORCH_CHECK(x.is_cuda() && q.is_cuda() && row_scale.is_cuda(), "tensors must be CUDA tensors");
    STD_TORCH_CHECK(x.dim() == 2, "x must be 2D");
    STD_TORCH_CHECK(is_half_or_bf16(x.scalar_type()), "x must be float16 or bfloat16");
    STD_TORCH_CHECK(q.scalar_type() == ScalarType::Char, "q must be int8");
    STD_TORCH_CHECK(row_scale.scalar_type() == ScalarType::Float, "row_scale must be float32");
    const int64_t M = x.size(0);
    const int64_t K = x.size(1);
    STD_TORCH_CHECK(q.dim() == 2 && q.size(0) == M && q.size(1) == K, "q must have the same shape as x");
    STD_TORCH_CHECK(row_scale.numel() == M, "row_scale must have M elements");
    STD_TORCH_CHECK(x.stride(0) == K && x.stride(1) == 1, "x must be contiguous");
    STD_TORCH_CHECK(q.stride(0) == K && q.stride(1) == 1, "q must be contiguous");
    STD_TORCH_CHECK(row_scale.is_contiguous(), "row_scale must be contiguous");
    STD_TORCH_CHECK(K % 256 == 0, "the contraction axis must be a multiple of the ConvRot group size (256)");
    const auto device = x.get_device_index();
    STD_TORCH_CHECK(q.get_device_index() == device && row_scale.get_device_index() == device, "q and row_scale must be on x's device");
    if (col_scale.has_value()) {
        STD_TORCH_CHECK(col_scale->scalar_type() == ScalarType::Float, "col_scale must be float32");
        STD_TORCH_CHECK(col_scale->numel() == K, "col_scale must have K elements");
        STD_TORCH_CHECK(col_scale->is_cuda() && col_scale->get_device_index() == device, "col_scale must be on x's device");
        STD_TORCH_CHECK(col_scale->is_contiguous() && aligned16(col_scale->const_data_ptr()), "col_scale must be contiguous and 16-byte aligned");
    }
    STD_TORCH_CHECK(aligned16(x.const_data_ptr()), "x data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(q.mutable_data_ptr()), "q data pointer must be 16-byte aligned");

    torch::stable::accelerator::DeviceGuard guard(device);
    const feather_stream_t stream = current_stream(device);
    const bool ok = launch_convrot_quantize(x.const_data_ptr(), col_scale.has_value() ? static_cast<const float*>(col_scale->const_data_ptr()) : nullptr,
                                            static_cast<int8_t*>(q.mutable_data_ptr()), static_cast<float*>(row_scale.mutable_data_ptr()), M, K,
                                            x.scalar_type() == ScalarType::Half ? 1 : 0, rotate, stream);
    STD_TORCH_CHECK(ok, "convrot_quantize launch failed");
}

void conv2d_3x3(const Tensor& x, const Tensor& w_prepacked, const std::optional<Tensor>& bias, Tensor& out, int64_t warps_m, int64_t warps_n,
                int64_t repeat_m, int64_t repeat_n, int64_t rows, bool prefetch) {
    STD_TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor");
    STD_TORCH_CHECK(w_prepacked.is_cuda(), "w_prepacked must be a CUDA tensor");
    STD_TORCH_CHECK(out.is_cuda(), "out must be a CUDA tensor");
    const auto device = x.get_device_index();
    STD_TORCH_CHECK(w_prepacked.get_device_index() == device, "w_prepacked must be on the same device as x");
    STD_TORCH_CHECK(out.get_device_index() == device, "out must be on the same device as x");
    const auto dtype = x.scalar_type();
    STD_TORCH_CHECK(is_half_or_bf16(dtype), "x must be float16 or bfloat16");
    STD_TORCH_CHECK(w_prepacked.scalar_type() == dtype, "w_prepacked must have x's dtype");
    STD_TORCH_CHECK(out.scalar_type() == dtype, "out must have x's dtype");
    STD_TORCH_CHECK(x.dim() == 4, "x must be 4D NCHW");
    STD_TORCH_CHECK(w_prepacked.dim() == 3, "w_prepacked must be 3D (K/8, C_out, 8)");
    STD_TORCH_CHECK(out.dim() == 4, "out must be 4D NCHW");

    const int64_t B = x.size(0);
    const int64_t C_in = x.size(1);
    const int64_t H = x.size(2);
    const int64_t W = x.size(3);
    const int64_t C_out = out.size(1);
    constexpr int64_t kIntMax = 2147483647;
    STD_TORCH_CHECK(B <= kIntMax && C_in <= kIntMax && C_out <= kIntMax && H <= kIntMax && W <= kIntMax, "conv2d_3x3: a dimension exceeds the 32-bit range");
    STD_TORCH_CHECK(out.size(0) == B && out.size(2) == H && out.size(3) == W, "out must be [B, C_out, H, W]");
    STD_TORCH_CHECK(w_prepacked.size(1) == C_out, "w_prepacked.shape[1] must equal C_out");
    STD_TORCH_CHECK(w_prepacked.size(2) == 8, "w_prepacked.shape[2] must be 8");
    STD_TORCH_CHECK(w_prepacked.size(0) == ((C_in + 15) / 16) * 18, "w_prepacked.shape[0] must equal ceil(C_in/16)*18");
    STD_TORCH_CHECK(C_in % 8 == 0, "conv2d_3x3 needs a multiple of 8 input channels");
    STD_TORCH_CHECK(x.stride(3) == 1 && x.stride(2) == W && x.stride(1) == H * W && x.stride(0) == C_in * H * W, "x must be contiguous NCHW");
    STD_TORCH_CHECK(out.stride(3) == 1 && out.stride(2) == W && out.stride(1) == H * W && out.stride(0) == C_out * H * W,
                    "out must be contiguous NCHW");
    STD_TORCH_CHECK(w_prepacked.stride(2) == 1 && w_prepacked.stride(1) == 8 && w_prepacked.stride(0) == C_out * 8, "w_prepacked must be contiguous");
    if (bias.has_value()) {
        STD_TORCH_CHECK(bias->is_cuda(), "bias must be a CUDA tensor");
        STD_TORCH_CHECK(bias->get_device_index() == device, "bias must be on the same device as x");
        STD_TORCH_CHECK(bias->scalar_type() == dtype, "bias must have x's dtype");
        STD_TORCH_CHECK(bias->numel() == C_out, "bias must have C_out elements");
        STD_TORCH_CHECK(bias->is_contiguous(), "bias must be contiguous");
    }

    torch::stable::accelerator::DeviceGuard guard(device);
    const feather_stream_t stream = current_stream(device);
    const void* const x_ptr = x.const_data_ptr();
    const void* const w_ptr = w_prepacked.const_data_ptr();
    const void* const bias_ptr = bias.has_value() ? bias->const_data_ptr() : nullptr;
    void* const out_ptr = out.mutable_data_ptr();
    STD_TORCH_CHECK(aligned16(x_ptr), "x data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(w_ptr), "w_prepacked data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(out_ptr), "out data pointer must be 16-byte aligned");
    STD_TORCH_CHECK(aligned16(bias_ptr == nullptr ? x_ptr : bias_ptr), "bias data pointer must be 16-byte aligned");

    const int rc = feather_conv3x3_launch(x_ptr, w_ptr, bias_ptr, out_ptr, static_cast<int>(B), static_cast<int>(C_in), static_cast<int>(C_out),
                                          static_cast<int>(H), static_cast<int>(W), bias.has_value() ? 1 : 0, static_cast<int>(warps_m),
                                          static_cast<int>(warps_n), static_cast<int>(repeat_m), static_cast<int>(repeat_n), static_cast<int>(rows),
                                          dtype == ScalarType::BFloat16 ? 1 : 0, prefetch ? 1 : 0, stream);
    STD_TORCH_CHECK(rc == 0, "conv2d_3x3: unsupported tile ", warps_m, "x", warps_n, " warp, ", repeat_m, "x", repeat_n, " repeat, ", rows, " rows");
}

}  // namespace

STABLE_TORCH_LIBRARY(feather_ops, m) {
    m.def(
        "scaled_mm(Tensor a, Tensor b_prepacked, Tensor? scale, Tensor? bias, Tensor(a!) c, int block_warps_m, int block_warps_n, "
        "int unroll_k, int repeat_m, int repeat_n, bool prefetch) -> ()");
    m.def(
        "scaled_mm_splitk(Tensor a, Tensor b_prepacked, Tensor? scale, Tensor? bias, Tensor(a!) c, Tensor(b!) partials, Tensor(c!) counters, "
        "int splits, int block_n=64) -> ()");
    m.def("interleave_slabs(Tensor slabs, Tensor(a!) out) -> ()");
    m.def(
        "int8_scaled_mm(Tensor a, Tensor b_prepacked, Tensor a_scale, Tensor? b_scale, Tensor? bias, Tensor(a!) c, bool transposed_b, "
        "int block_warps_m, int block_warps_n, int unroll_k, int repeat_m, int repeat_n) -> ()");
    m.def("int8_scaled_mm_plain(Tensor a, Tensor weight, Tensor a_scale, Tensor? b_scale, Tensor? bias, Tensor(a!) c, bool transposed_b) -> ()");
    m.def("convrot_quantize(Tensor x, Tensor? col_scale, Tensor(a!) q, Tensor(b!) row_scale, bool rotate) -> ()");
    m.def(
        "conv2d_3x3(Tensor x, Tensor w_prepacked, Tensor? bias, Tensor(a!) out, int warps_m, int warps_n, int repeat_m, int repeat_n, "
        "int rows, bool prefetch) -> ()");
}

STABLE_TORCH_LIBRARY_IMPL(feather_ops, CUDA, m) {
    m.impl("scaled_mm", TORCH_BOX(&scaled_mm));
    m.impl("scaled_mm_splitk", TORCH_BOX(&scaled_mm_splitk));
    m.impl("interleave_slabs", TORCH_BOX(&interleave_slabs));
    m.impl("int8_scaled_mm", TORCH_BOX(&int8_scaled_mm));
    m.impl("int8_scaled_mm_plain", TORCH_BOX(&int8_scaled_mm_plain));
    m.impl("convrot_quantize", TORCH_BOX(&convrot_quantize));
    m.impl("conv2d_3x3", TORCH_BOX(&conv2d_3x3));
}

extern "C" PyObject* PyInit__C(void) {
    static PyModuleDef module = {PyModuleDef_HEAD_INIT, "_C", nullptr, -1, nullptr, nullptr, nullptr, nullptr, nullptr};
    return PyModule_Create(&module);
}
