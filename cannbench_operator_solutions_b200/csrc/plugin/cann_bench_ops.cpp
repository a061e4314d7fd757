// torch operator plugin: registers the reference catalog's operator schemas in
// namespace cann_bench and implements them for the CUDA dispatch key on top of
// the C-ABI in include/w8a8ffn.h.
//
// Schemas, output allocation ("meta") and argument checks mirror the reference
// plugins one to one:
//   dynamic_quant               operators/dynamicquant/csrc/ops/dynamic_quant/op_plugin/dynamic_quant_plugin.cpp:28-92
//   add_rms_norm_dynamic_quant  operators/addrmsnormdynamicquant/csrc/ops/add_rms_norm_dynamic_quant/op_plugin/add_rms_norm_dynamic_quant_plugin.cpp:30-119
//   quant_matmul                operators/quantmatmul/csrc/ops/quant_matmul/op_plugin/quant_matmul_plugin.cpp:46-272
//   grouped_matmul_swiglu_quant operators/groupedmatmulswigluquant/csrc/ops/grouped_matmul_swiglu_quant/op_plugin/gmsq_plugin.cpp:38-150
//   grouped_matmul              operators/groupedmatmul/csrc/ops/grouped_matmul/op_plugin/grouped_matmul_plugin.cpp:40-190
//   moe_re_routing              operators/moererouting/csrc/ops/moe_re_routing/op_plugin/moe_re_routing_plugin.cpp:32-170
//   dequant_swiglu_quant        operators/dequantswigluquant/csrc/ops/dequant_swiglu_quant/op_plugin/dqsq_plugin.cpp:31-160
//   moe_gating_top_k_softmax    operators/moegatingtopksoftmax/csrc/ops/moe_gating_top_k_softmax/op_plugin/moe_gating_plugin.cpp:28-120
//   moe_finalize_routing        operators/moefinalizerouting/csrc/ops/moe_finalize_routing/op_plugin/moe_finalize_routing_plugin.cpp:31-237
// The NPU plugins enqueue their launchers with OpCommand::RunOpApi on the
// current NPU stream; here the C-ABI call is enqueued on the current CUDA
// stream.  The plugin only unpacks tensors: all arithmetic is in the library.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <string>
#include <tuple>
#include <vector>

#include "../../../include/w8a8ffn.h"

namespace cann_bench {

static void check_status(int rc, const char* op)
{
    TORCH_CHECK(rc == W8A8_OK, op, ": ", w8a8_status_string(rc), " (status ", rc, ")");
}

static int dtype_code(const torch::Tensor& t)
{
    switch (t.scalar_type()) {
    case torch::kFloat16:
        return W8A8_DT_F16;
    case torch::kBFloat16:
        return W8A8_DT_BF16;
    case torch::kFloat32:
        return W8A8_DT_F32;
    case torch::kChar:
        return W8A8_DT_I8;
    default:
        TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
    }
    return -1;
}

static void* stream_of(const torch::Tensor& t)
{
    return static_cast<void*>(at::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

// ----------------------------------------------------------------- dynamic_quant
static std::tuple<torch::Tensor, torch::Tensor> dynamic_quant_meta(const torch::Tensor& x)
{
    TORCH_CHECK(x.dim() >= 2, "dynamic_quant requires a tensor with rank >= 2.");
    TORCH_CHECK(x.scalar_type() == torch::kFloat16 || x.scalar_type() == torch::kBFloat16,
                "dynamic_quant only supports float16 / bfloat16 inputs.");
    std::vector<int64_t> scale_shape(x.sizes().begin(), x.sizes().end() - 1);
    auto y = torch::empty_like(x, x.options().dtype(torch::kChar));
    auto scale = torch::empty(scale_shape, x.options().dtype(torch::kFloat));
    return std::make_tuple(y, scale);
}

static std::tuple<torch::Tensor, torch::Tensor> dynamic_quant_cuda(const torch::Tensor& x)
{
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    auto xc = x.contiguous();
    auto outs = dynamic_quant_meta(xc);
    const int64_t N = xc.size(-1);
    TORCH_CHECK(N > 0, "dynamic_quant requires a non-zero last dimension.");
    const int64_t M = xc.numel() / N;
    if (M <= 0) {
        return outs;
    }
    check_status(w8a8_dynamic_quant(xc.data_ptr(), static_cast<int8_t*>(std::get<0>(outs).data_ptr()),
                                    static_cast<float*>(std::get<1>(outs).data_ptr()), M, N, dtype_code(xc), 0,
                                    stream_of(xc)),
                 "dynamic_quant");
    return outs;
}

// ------------------------------------------------------ add_rms_norm_dynamic_quant
static std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> ardq_meta(const torch::Tensor& x1,
                                                                         const torch::Tensor& x2,
                                                                         const torch::Tensor& gamma, double epsilon)
{
    (void)epsilon;
    TORCH_CHECK(x1.dim() >= 1, "add_rms_norm_dynamic_quant: x1 must have at least one dimension.");
    TORCH_CHECK(x1.sizes() == x2.sizes(), "add_rms_norm_dynamic_quant: x1 and x2 must share a shape.");
    TORCH_CHECK(gamma.dim() == 1 && gamma.size(0) == x1.size(-1),
                "add_rms_norm_dynamic_quant: gamma must be 1-D with size == x1.size(-1).");
    TORCH_CHECK(gamma.scalar_type() == x1.scalar_type(),
                "add_rms_norm_dynamic_quant: gamma dtype must match x1 dtype.");
    auto y = torch::empty_like(x1, x1.options().dtype(torch::kChar));
    auto x_out = torch::empty_like(x1);
    std::vector<int64_t> scale_shape(x1.sizes().begin(), x1.sizes().end() - 1);
    auto scale = torch::empty(scale_shape, x1.options().dtype(torch::kFloat));
    return std::make_tuple(y, x_out, scale);
}

static std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> ardq_cuda(const torch::Tensor& x1,
                                                                         const torch::Tensor& x2,
                                                                         const torch::Tensor& gamma, double epsilon)
{
    const c10::cuda::OptionalCUDAGuard guard(x1.device());
    auto x1c = x1.contiguous();
    auto x2c = x2.contiguous();
    auto gc = gamma.contiguous();
    auto outs = ardq_meta(x1c, x2c, gc, epsilon);
    const int64_t N = x1c.size(-1);
    if (x1c.numel() == 0 || N <= 0) {
        return outs;
    }
    TORCH_CHECK(x1c.scalar_type() == torch::kFloat16 || x1c.scalar_type() == torch::kBFloat16,
                "add_rms_norm_dynamic_quant: only float16/bfloat16 inputs are supported.");
    TORCH_CHECK(x2c.scalar_type() == x1c.scalar_type(), "add_rms_norm_dynamic_quant: x2 dtype must match x1 dtype.");
    TORCH_CHECK(N <= 16384, "add_rms_norm_dynamic_quant: row length must not exceed 16384.");
    const int64_t rows = x1c.numel() / N;
    check_status(w8a8_add_rms_norm_dynamic_quant(x1c.data_ptr(), x2c.data_ptr(), gc.data_ptr(),
                                                 static_cast<int8_t*>(std::get<0>(outs).data_ptr()),
                                                 std::get<1>(outs).data_ptr(),
                                                 static_cast<float*>(std::get<2>(outs).data_ptr()), rows, N,
                                                 static_cast<float>(epsilon), dtype_code(x1c), 0, stream_of(x1c)),
                 "add_rms_norm_dynamic_quant");
    return outs;
}

// ------------------------------------------------------------------ quant_matmul
static torch::Tensor quant_matmul_meta(const torch::Tensor& x1, const torch::Tensor& x2, const torch::Tensor& scale,
                                       const c10::optional<torch::Tensor>& offset,
                                       const c10::optional<torch::Tensor>& pertoken_scale,
                                       const c10::optional<torch::Tensor>& bias,
                                       const c10::optional<std::string>& output_dtype)
{
    (void)scale;
    (void)offset;
    (void)pertoken_scale;
    (void)bias;
    TORCH_CHECK(x1.dim() >= 2 && x2.dim() >= 2, "quant_matmul requires inputs of rank >= 2.");
    TORCH_CHECK(x1.size(-1) == x2.size(-2), "quant_matmul requires x1.size(-1) == x2.size(-2).");
    const bool bf16out = output_dtype.has_value() && output_dtype.value() == "bfloat16";
    std::vector<int64_t> out_shape(x1.sizes().begin(), x1.sizes().end() - 1);
    out_shape.push_back(x2.size(-1));
    return torch::empty(out_shape, x1.options().dtype(bf16out ? torch::kBFloat16 : torch::kFloat16));
}

static torch::Tensor quant_matmul_cuda(const torch::Tensor& x1, const torch::Tensor& x2, const torch::Tensor& scale,
                                       const c10::optional<torch::Tensor>& offset,
                                       const c10::optional<torch::Tensor>& pertoken_scale,
                                       const c10::optional<torch::Tensor>& bias,
                                       const c10::optional<std::string>& output_dtype)
{
    const c10::cuda::OptionalCUDAGuard guard(x1.device());
    TORCH_CHECK(x1.scalar_type() == torch::kChar && x2.scalar_type() == torch::kChar,
                "quant_matmul requires int8 x1 and x2.");
    TORCH_CHECK(x1.is_contiguous() && x2.is_contiguous() && scale.is_contiguous(),
                "quant_matmul requires contiguous x1/x2/scale.");
    TORCH_CHECK(scale.scalar_type() == torch::kFloat32 || scale.scalar_type() == torch::kBFloat16,
                "quant_matmul requires float32 or bfloat16 scale.");
    TORCH_CHECK(x1.dim() >= 2 && x2.dim() >= 2 && x1.dim() == x2.dim(), "quant_matmul expects equal ranks >= 2.");
    TORCH_CHECK(x1.size(-1) == x2.size(-2), "quant_matmul requires x1.size(-1) == x2.size(-2).");
    const int64_t K = x1.size(-1), M = x1.size(-2), N = x2.size(-1);
    TORCH_CHECK(K > 0 && M > 0 && N > 0, "quant_matmul requires non-empty shapes.");
    int64_t batch = 1;
    for (int64_t d = 0; d + 2 < x1.dim(); ++d) {
        TORCH_CHECK(x1.size(d) == x2.size(d), "quant_matmul expects matching leading batch dimensions.");
        batch *= x1.size(d);
    }
    auto out = quant_matmul_meta(x1, x2, scale, offset, pertoken_scale, bias, output_dtype);
    const bool bf16out = out.scalar_type() == torch::kBFloat16;

    int64_t flags = 0;
    TORCH_CHECK(scale.numel() == 1 || scale.numel() == N, "quant_matmul expects scale length 1 or n.");
    if (scale.numel() > 1) {
        flags |= W8A8_QM_SCALE_PERCHAN;
    }
    if (scale.scalar_type() == torch::kBFloat16) {
        flags |= W8A8_QM_SCALE_BF16;
    }
    const bool has_offset = offset.has_value() && offset->defined();
    if (has_offset) {
        TORCH_CHECK(offset->scalar_type() == torch::kFloat32 && offset->is_contiguous(),
                    "quant_matmul requires float32 contiguous offset.");
        TORCH_CHECK(offset->numel() == 1 || offset->numel() == N, "quant_matmul expects offset length 1 or n.");
        flags |= W8A8_QM_HAS_OFFSET;
        if (offset->numel() > 1) {
            flags |= W8A8_QM_OFFSET_PERCHAN;
        }
    }
    const bool has_pt = pertoken_scale.has_value() && pertoken_scale->defined();
    if (has_pt) {
        TORCH_CHECK(pertoken_scale->scalar_type() == torch::kFloat32 && pertoken_scale->is_contiguous(),
                    "quant_matmul requires float32 contiguous pertoken_scale.");
        TORCH_CHECK(pertoken_scale->numel() == M, "quant_matmul expects pertoken_scale length m.");
        flags |= W8A8_QM_HAS_PT;
    }
    const bool has_bias = bias.has_value() && bias->defined();
    int64_t bias_batch_stride = 0;
    if (has_bias) {
        TORCH_CHECK(bias->is_contiguous(), "quant_matmul requires contiguous bias.");
        int64_t kind = W8A8_QM_BIAS_NONE;
        switch (bias->scalar_type()) {
        case torch::kInt32:
            kind = W8A8_QM_BIAS_I32;
            break;
        case torch::kFloat16:
            kind = W8A8_QM_BIAS_F16;
            break;
        case torch::kBFloat16:
            kind = W8A8_QM_BIAS_BF16;
            break;
        case torch::kFloat32:
            kind = W8A8_QM_BIAS_F32;
            break;
        default:
            TORCH_CHECK(false, "quant_matmul unsupported bias dtype: ", bias->scalar_type());
        }
        bool per_chan;
        if (bias->dim() == 3 && bias->size(1) == 1 && bias->size(2) == N && batch > 1 && bias->size(0) == batch) {
            bias_batch_stride = N;
            per_chan = N > 1;
        } else {
            TORCH_CHECK(bias->numel() == 1 || bias->numel() == N, "quant_matmul expects bias length 1 or n.");
            per_chan = bias->numel() > 1;
        }
        flags |= kind << W8A8_QM_BIAS_SHIFT;
        if (per_chan) {
            flags |= W8A8_QM_BIAS_PERCHAN;
        }
    }
    if (batch > 1) {
        flags |= W8A8_QM_PT_MOD_M;
    }
    check_status(w8a8_quant_matmul(static_cast<const int8_t*>(x1.data_ptr()), static_cast<const int8_t*>(x2.data_ptr()),
                                   scale.data_ptr(), has_offset ? static_cast<const float*>(offset->data_ptr()) : nullptr,
                                   has_pt ? static_cast<const float*>(pertoken_scale->data_ptr()) : nullptr,
                                   has_bias ? bias->data_ptr() : nullptr, out.data_ptr(), batch, M, N, K, flags,
                                   bf16out ? W8A8_DT_BF16 : W8A8_DT_F16, W8A8_W_KN, bias_batch_stride, stream_of(x1)),
                 "quant_matmul");
    return out;
}

// --------------------------------------------------- grouped_matmul_swiglu_quant
static std::vector<int64_t> collect_ends(c10::List<int64_t> group_list, int64_t E, int64_t M, const char* op)
{
    TORCH_CHECK(static_cast<int64_t>(group_list.size()) == E, op, ": group_list length must equal the expert count");
    std::vector<int64_t> ends(static_cast<size_t>(E));
    int64_t prev = 0;
    for (int64_t g = 0; g < E; ++g) {
        const int64_t v = group_list[static_cast<size_t>(g)];
        TORCH_CHECK(v >= prev && v <= M, op, ": group_list must be a cumsum <= M");
        ends[static_cast<size_t>(g)] = v;
        prev = v;
    }
    TORCH_CHECK(prev == M, op, ": group_list[-1] must equal M");
    return ends;
}

static std::tuple<torch::Tensor, torch::Tensor> gmsq_meta(const torch::Tensor& x, const torch::Tensor& weight,
                                                          const torch::Tensor& weight_scale,
                                                          const torch::Tensor& x_scale, c10::List<int64_t> group_list)
{
    (void)weight_scale;
    (void)x_scale;
    (void)group_list;
    TORCH_CHECK(x.dim() == 2, "grouped_matmul_swiglu_quant: x must be 2D [M, K]");
    TORCH_CHECK(weight.dim() == 3, "grouped_matmul_swiglu_quant: weight must be 3D [E, K, N]");
    const int64_t M = x.size(0);
    const int64_t N = weight.size(2);
    TORCH_CHECK(N % 2 == 0, "grouped_matmul_swiglu_quant: N must be even");
    auto y = torch::empty({M, N / 2}, x.options().dtype(torch::kChar));
    auto y_scale = torch::empty({M}, x.options().dtype(torch::kFloat32));
    return std::make_tuple(y, y_scale);
}

static std::tuple<torch::Tensor, torch::Tensor> gmsq_cuda(const torch::Tensor& x, const torch::Tensor& weight,
                                                          const torch::Tensor& weight_scale,
                                                          const torch::Tensor& x_scale, c10::List<int64_t> group_list)
{
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    TORCH_CHECK(x.scalar_type() == torch::kChar, "grouped_matmul_swiglu_quant: x must be int8");
    TORCH_CHECK(weight.scalar_type() == torch::kChar, "grouped_matmul_swiglu_quant: weight must be int8");
    TORCH_CHECK(weight_scale.scalar_type() == torch::kFloat, "grouped_matmul_swiglu_quant: weight_scale must be float32");
    TORCH_CHECK(x_scale.scalar_type() == torch::kFloat, "grouped_matmul_swiglu_quant: x_scale must be float32");
    auto xc = x.contiguous();
    auto wc = weight.contiguous();
    auto wsc = weight_scale.contiguous();
    auto xsc = x_scale.contiguous();
    auto outs = gmsq_meta(xc, wc, wsc, xsc, group_list);
    const int64_t M = xc.size(0), K = xc.size(1), E = wc.size(0), N = wc.size(2);
    if (M == 0 || N == 0 || E == 0) {
        return outs;
    }
    TORCH_CHECK(wc.size(1) == K, "grouped_matmul_swiglu_quant: K mismatch between x and weight");
    TORCH_CHECK(xsc.numel() == M, "grouped_matmul_swiglu_quant: x_scale must have M elements");
    TORCH_CHECK(wsc.dim() == 2 && wsc.size(0) == E && wsc.size(1) == N,
                "grouped_matmul_swiglu_quant: weight_scale must be [E, N]");
    const std::vector<int64_t> ends = collect_ends(group_list, E, M, "grouped_matmul_swiglu_quant");
    const size_t ws_bytes = w8a8_grouped_matmul_swiglu_quant_workspace_size(M, K, N, E);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes)}, xc.options().dtype(torch::kUInt8));
    check_status(w8a8_grouped_matmul_swiglu_quant(
                     static_cast<const int8_t*>(xc.data_ptr()), static_cast<const int8_t*>(wc.data_ptr()),
                     static_cast<const float*>(wsc.data_ptr()), static_cast<const float*>(xsc.data_ptr()),
                     static_cast<int8_t*>(std::get<0>(outs).data_ptr()),
                     static_cast<float*>(std::get<1>(outs).data_ptr()), M, K, N, E, ends.data(), 0, W8A8_W_KN, 0,
                     ws.data_ptr(), ws_bytes, stream_of(xc)),
                 "grouped_matmul_swiglu_quant");
    return outs;
}

// ---------------------------------------------------------------- grouped_matmul
static c10::List<torch::Tensor> make_outputs(const torch::Tensor& y, const std::vector<int64_t>& ends,
                                             int64_t split_item)
{
    c10::List<torch::Tensor> out;
    if (split_item == 0 || split_item == 1) {
        int64_t s = 0;
        for (const int64_t e : ends) {
            out.push_back(y.narrow(0, s, e - s));
            s = e;
        }
    } else {
        out.push_back(y);
    }
    return out;
}

static c10::List<torch::Tensor> grouped_matmul_meta(const torch::Tensor& x, const torch::Tensor& weight,
                                                    c10::List<int64_t> group_list,
                                                    const c10::optional<torch::Tensor>& bias, int64_t split_item,
                                                    bool transpose_weight,
                                                    const c10::optional<torch::Tensor>& x_scale,
                                                    const c10::optional<torch::Tensor>& weight_scale)
{
    (void)bias;
    (void)weight_scale;
    TORCH_CHECK(x.dim() == 2, "grouped_matmul: x must be 2D [M, K]");
    TORCH_CHECK(weight.dim() == 3, "grouped_matmul: weight must be 3D [E, K, N] or [E, N, K]");
    const int64_t M = x.size(0);
    const int64_t E = weight.size(0);
    const int64_t N = transpose_weight ? weight.size(1) : weight.size(2);
    const std::vector<int64_t> ends = collect_ends(group_list, E, M, "grouped_matmul");
    const bool quant = x_scale.has_value() && x_scale->defined();
    auto y = torch::empty({M, N}, quant ? x.options().dtype(torch::kBFloat16) : x.options());
    return make_outputs(y, ends, split_item);
}

static c10::List<torch::Tensor> grouped_matmul_cuda(const torch::Tensor& x, const torch::Tensor& weight,
                                                    c10::List<int64_t> group_list,
                                                    const c10::optional<torch::Tensor>& bias, int64_t split_item,
                                                    bool transpose_weight,
                                                    const c10::optional<torch::Tensor>& x_scale,
                                                    const c10::optional<torch::Tensor>& weight_scale)
{
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    auto xc = x.contiguous();
    auto wc = weight.contiguous();
    const int64_t M = xc.size(0), K = xc.size(1), E = wc.size(0);
    TORCH_CHECK(E >= 1, "grouped_matmul: weight must contain at least one expert");
    const int64_t N = transpose_weight ? wc.size(1) : wc.size(2);
    const int64_t k_stored = transpose_weight ? wc.size(2) : wc.size(1);
    TORCH_CHECK(k_stored == K, "grouped_matmul: K dimension mismatch between x and weight");
    TORCH_CHECK(xc.scalar_type() == wc.scalar_type(), "grouped_matmul: x and weight must share a dtype");
    const std::vector<int64_t> ends = collect_ends(group_list, E, M, "grouped_matmul");
    const int dt = dtype_code(xc);
    const bool quant = dt == W8A8_DT_I8;
    torch::Tensor xs, wsc;
    if (quant) {
        TORCH_CHECK(x_scale.has_value() && weight_scale.has_value(),
                    "grouped_matmul: int8 inputs need x_scale and weight_scale");
        xs = x_scale->contiguous();
        wsc = weight_scale->contiguous();
        TORCH_CHECK(xs.scalar_type() == torch::kFloat && xs.numel() == M, "grouped_matmul: x_scale must be fp32 [M]");
        TORCH_CHECK(wsc.scalar_type() == torch::kFloat && wsc.numel() == E * N,
                    "grouped_matmul: weight_scale must be fp32 [E, N]");
    } else {
        TORCH_CHECK(!(x_scale.has_value() && x_scale->defined()) && !(weight_scale.has_value() && weight_scale->defined()),
                    "grouped_matmul: scales are only valid with int8 inputs");
    }
    const bool has_bias = bias.has_value() && bias->defined();
    torch::Tensor bc;
    if (has_bias) {
        bc = bias->contiguous();
        TORCH_CHECK(bc.numel() == E * N, "grouped_matmul: bias must have shape [E, N]");
    }
    auto y = torch::empty({M, N}, quant ? xc.options().dtype(torch::kBFloat16) : xc.options());
    if (M > 0) {
        const size_t ws_bytes = w8a8_grouped_matmul_workspace_size(M, N, K, E);
        auto ws = torch::empty({static_cast<int64_t>(ws_bytes)}, xc.options().dtype(torch::kUInt8));
        check_status(w8a8_grouped_matmul(xc.data_ptr(), wc.data_ptr(), has_bias ? bc.data_ptr() : nullptr, y.data_ptr(),
                                         quant ? static_cast<const float*>(xs.data_ptr()) : nullptr,
                                         quant ? static_cast<const float*>(wsc.data_ptr()) : nullptr, M, N, K, E,
                                         ends.data(), 0, dt, has_bias ? dtype_code(bc) : dt, dtype_code(y),
                                         transpose_weight ? W8A8_W_NK : W8A8_W_KN, ws.data_ptr(), ws_bytes,
                                         stream_of(xc)),
                     "grouped_matmul");
    }
    return make_outputs(y, ends, split_item);
}

// ---------------------------------------------------------------- moe_re_routing
using RrOut = std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>;

static RrOut moe_re_routing_meta(const torch::Tensor& tokens, const torch::Tensor& counts,
                                 const c10::optional<torch::Tensor>& scales, int64_t expert_token_num_type,
                                 int64_t idx_type)
{
    (void)scales;
    (void)expert_token_num_type;
    (void)idx_type;
    TORCH_CHECK(tokens.dim() == 2, "moe_re_routing: tokens must be 2D (A, H).");
    TORCH_CHECK(counts.dim() == 2, "moe_re_routing: expert_token_num_per_rank must be 2D (N, E).");
    const int64_t a = tokens.size(0);
    return std::make_tuple(torch::empty({a, tokens.size(1)}, tokens.options()),
                           torch::empty({a}, tokens.options().dtype(torch::kFloat)),
                           torch::empty({a}, tokens.options().dtype(torch::kInt)),
                           torch::empty({counts.size(1)}, counts.options()));
}

static RrOut moe_re_routing_cuda(const torch::Tensor& tokens, const torch::Tensor& counts,
                                 const c10::optional<torch::Tensor>& scales, int64_t expert_token_num_type,
                                 int64_t idx_type)
{
    TORCH_CHECK(idx_type == 0, "moe_re_routing: only gather index mode (idx_type == 0) is supported.");
    const c10::cuda::OptionalCUDAGuard guard(tokens.device());
    auto tok = tokens.contiguous();
    auto cnt = counts.contiguous();
    torch::Tensor scl;
    const bool has_scales = scales.has_value() && scales->defined();
    if (has_scales) {
        scl = scales->contiguous();
        TORCH_CHECK(scl.scalar_type() == torch::kFloat, "moe_re_routing: per_token_scales must be float32.");
    }
    auto outs = moe_re_routing_meta(tok, cnt, scales, expert_token_num_type, idx_type);
    const int64_t a = tok.size(0), h = tok.size(1), n = cnt.size(0), e = cnt.size(1);
    if (a <= 0 || h <= 0 || n <= 0 || e <= 0) {
        return outs;
    }
    TORCH_CHECK(tok.scalar_type() == torch::kFloat16 || tok.scalar_type() == torch::kBFloat16 ||
                    tok.scalar_type() == torch::kChar,
                "moe_re_routing: unsupported tokens dtype.");
    TORCH_CHECK(cnt.scalar_type() == torch::kInt || cnt.scalar_type() == torch::kLong,
                "moe_re_routing: unsupported expert_token_num_per_rank dtype.");
    TORCH_CHECK(cnt.is_cuda(), "moe_re_routing: expert_token_num_per_rank must be on the tokens' device.");
    if (has_scales) {
        TORCH_CHECK(scl.numel() == a, "moe_re_routing: per_token_scales must have A elements.");
    }
    const size_t ws_bytes = w8a8_moe_re_routing_workspace_size(a, n, e);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes)}, tok.options().dtype(torch::kByte));
    check_status(w8a8_moe_re_routing(tok.data_ptr(), cnt.data_ptr(),
                                     has_scales ? static_cast<const float*>(scl.data_ptr()) : nullptr,
                                     std::get<0>(outs).data_ptr(), static_cast<float*>(std::get<1>(outs).data_ptr()),
                                     static_cast<int32_t*>(std::get<2>(outs).data_ptr()),
                                     std::get<3>(outs).data_ptr(), a, h * static_cast<int64_t>(tok.element_size()), n,
                                     e, static_cast<int>(cnt.element_size()), ws.data_ptr(), ws_bytes,
                                     stream_of(tok)),
                 "moe_re_routing");
    return outs;
}

// ---------------------------------------------------------- moe_finalize_routing
static bool present(const c10::optional<torch::Tensor>& t)
{
    return t.has_value() && t->defined();
}

static void mfr_shape(const torch::Tensor& epr, const torch::Tensor& esdr, const c10::optional<torch::Tensor>& scales,
                      int64_t& num_rows, int64_t& K, int64_t& H)
{
    TORCH_CHECK(epr.dim() >= 2, "moe_finalize_routing: expanded_permuted_rows must have rank >= 2.");
    TORCH_CHECK(esdr.scalar_type() == torch::kInt, "moe_finalize_routing: expanded_src_to_dst_row must be int32.");
    H = epr.size(-1);
    K = 1;
    if (present(scales)) {
        TORCH_CHECK(scales->dim() == 2, "moe_finalize_routing: scales must be 2-D (NUM_ROWS, K).");
        K = scales->size(1);
    }
    TORCH_CHECK(K > 0, "moe_finalize_routing: K must be positive.");
    TORCH_CHECK(esdr.numel() % K == 0, "moe_finalize_routing: expanded_src_to_dst_row length must be K*NUM_ROWS.");
    num_rows = esdr.numel() / K;
}

static torch::Tensor mfr_meta(const torch::Tensor& epr, const torch::Tensor& esdr, c10::optional<torch::Tensor> skip1,
                              c10::optional<torch::Tensor> skip2, c10::optional<torch::Tensor> bias,
                              c10::optional<torch::Tensor> scales, c10::optional<torch::Tensor> expert,
                              int64_t drop_pad_mode)
{
    (void)skip1;
    (void)skip2;
    (void)bias;
    (void)expert;
    (void)drop_pad_mode;
    int64_t num_rows = 0, K = 1, H = 0;
    mfr_shape(epr, esdr, scales, num_rows, K, H);
    return torch::empty({num_rows, H}, epr.options());
}

static torch::Tensor mfr_cuda(const torch::Tensor& rows, const torch::Tensor& src_to_dst,
                              c10::optional<torch::Tensor> skip1, c10::optional<torch::Tensor> skip2,
                              c10::optional<torch::Tensor> bias, c10::optional<torch::Tensor> scales,
                              c10::optional<torch::Tensor> expert, int64_t drop_pad_mode)
{
    const auto t = rows.scalar_type();
    TORCH_CHECK(t == torch::kFloat16 || t == torch::kFloat32 || t == torch::kBFloat16,
                "moe_finalize_routing: expanded_permuted_rows must be float16 / float32 / bfloat16.");
    const c10::cuda::OptionalCUDAGuard guard(rows.device());
    auto epr = rows.contiguous();
    auto esdr = src_to_dst.contiguous();
    int64_t num_rows = 0, K = 1, H = 0;
    mfr_shape(epr, esdr, scales, num_rows, K, H);
    auto out = torch::empty({num_rows, H}, epr.options());
    if (num_rows <= 0 || H <= 0) {
        return out;
    }
    const bool has_scales = present(scales);
    const bool has_expert = present(expert);
    const bool has_bias = present(bias) && has_expert;
    if (has_bias) {
        TORCH_CHECK(bias->size(1) == H, "moe_finalize_routing: bias head dim must equal H.");
        TORCH_CHECK(bias->scalar_type() == t, "moe_finalize_routing: bias must have the rows' dtype.");
        TORCH_CHECK(expert->scalar_type() == torch::kInt, "moe_finalize_routing: expert_for_source_row must be int32.");
    }
    TORCH_CHECK(!present(skip1) || skip1->scalar_type() == t, "moe_finalize_routing: skip1 must have the rows' dtype.");
    TORCH_CHECK(!present(skip2) || skip2->scalar_type() == t, "moe_finalize_routing: skip2 must have the rows' dtype.");
    torch::Tensor s1, s2, bs, sc, ex;
    if (present(skip1)) {
        s1 = skip1->contiguous();
    }
    if (present(skip2)) {
        s2 = skip2->contiguous();
    }
    if (has_bias) {
        bs = bias->contiguous();
        ex = expert->contiguous();
    }
    int sdt = dtype_code(epr);
    if (has_scales) {
        sc = scales->contiguous();
        const auto st = sc.scalar_type();
        TORCH_CHECK(st == torch::kFloat16 || st == torch::kFloat32 || st == torch::kBFloat16,
                    "moe_finalize_routing: unsupported dtype combination for expanded_permuted_rows / scales.");
        sdt = dtype_code(sc);
    }
    const int64_t mode = drop_pad_mode < 0 ? 0 : (drop_pad_mode > 3 ? 3 : drop_pad_mode);
    check_status(w8a8_moe_finalize_routing(epr.data_ptr(), static_cast<const int32_t*>(esdr.data_ptr()),
                                           s1.defined() ? s1.data_ptr() : nullptr,
                                           s2.defined() ? s2.data_ptr() : nullptr,
                                           has_bias ? bs.data_ptr() : nullptr, has_scales ? sc.data_ptr() : nullptr,
                                           has_bias ? static_cast<const int32_t*>(ex.data_ptr()) : nullptr,
                                           out.data_ptr(), num_rows, H, K, has_bias ? bs.size(0) : 0,
                                           epr.numel() / H, static_cast<int>(mode), dtype_code(epr), sdt,
                                           stream_of(epr)),
                 "moe_finalize_routing");
    return out;
}

// ------------------------------------------------------ moe_gating_top_k_softmax
using GateOut = std::tuple<torch::Tensor, torch::Tensor, torch::Tensor>;

static GateOut gating_meta(const torch::Tensor& x, const c10::optional<torch::Tensor>& finished, int64_t k)
{
    TORCH_CHECK(x.scalar_type() == torch::kFloat32 || x.scalar_type() == torch::kFloat16 ||
                    x.scalar_type() == torch::kBFloat16,
                "cann_bench.moe_gating_top_k_softmax only supports float32, float16 and bfloat16 inputs.");
    TORCH_CHECK(x.dim() >= 2, "cann_bench.moe_gating_top_k_softmax requires a tensor with rank >= 2.");
    const int64_t inner = x.size(-1);
    TORCH_CHECK(inner > 0, "cann_bench.moe_gating_top_k_softmax requires a non-empty last dimension.");
    TORCH_CHECK(k > 0 && k <= inner, "cann_bench.moe_gating_top_k_softmax requires 0 < k <= x.size(-1).");
    if (present(finished)) {
        TORCH_CHECK(finished->scalar_type() == torch::kBool,
                    "cann_bench.moe_gating_top_k_softmax requires a bool 'finished' tensor.");
    }
    std::vector<int64_t> shape(x.sizes().begin(), x.sizes().end() - 1);
    shape.push_back(k);
    return std::make_tuple(torch::empty(shape, x.options()), torch::empty(shape, x.options().dtype(torch::kInt)),
                           torch::empty(shape, x.options().dtype(torch::kInt)));
}

static GateOut gating_cuda(const torch::Tensor& x, const c10::optional<torch::Tensor>& finished, int64_t k)
{
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    auto xc = x.contiguous();
    auto outs = gating_meta(xc, finished, k);
    const int64_t inner = xc.size(-1);
    const int64_t rows = xc.numel() / inner;
    TORCH_CHECK(rows > 0, "cann_bench.moe_gating_top_k_softmax requires at least one row.");
    torch::Tensor fin;
    if (present(finished)) {
        fin = finished->contiguous();
        TORCH_CHECK(fin.numel() == rows, "cann_bench.moe_gating_top_k_softmax: finished must have numel == rows.");
    }
    check_status(w8a8_moe_gating_top_k_softmax(xc.data_ptr(),
                                               fin.defined() ? static_cast<const uint8_t*>(fin.data_ptr()) : nullptr,
                                               std::get<0>(outs).data_ptr(),
                                               static_cast<int32_t*>(std::get<1>(outs).data_ptr()),
                                               static_cast<int32_t*>(std::get<2>(outs).data_ptr()), rows, inner, k,
                                               dtype_code(xc), stream_of(xc)),
                 "moe_gating_top_k_softmax");
    return outs;
}

// ---------------------------------------------------------- dequant_swiglu_quant
static std::tuple<torch::Tensor, torch::Tensor> dqsq_meta(const torch::Tensor& x,
                                                          const c10::optional<torch::Tensor>& weight_scale,
                                                          const c10::optional<torch::Tensor>& activation_scale,
                                                          const c10::optional<torch::Tensor>& quant_scale,
                                                          bool activate_left)
{
    (void)weight_scale;
    (void)activation_scale;
    (void)quant_scale;
    (void)activate_left;
    TORCH_CHECK(x.dim() == 2, "dequant_swiglu_quant requires a 2D input [TokensNum, 2H].");
    TORCH_CHECK(x.size(1) % 2 == 0, "dequant_swiglu_quant requires an even last dimension.");
    return std::make_tuple(torch::empty({x.size(0), x.size(1) / 2}, x.options().dtype(torch::kChar)),
                           torch::empty({x.size(0)}, x.options().dtype(torch::kFloat)));
}

static std::tuple<torch::Tensor, torch::Tensor> dqsq_cuda(const torch::Tensor& x,
                                                          const c10::optional<torch::Tensor>& weight_scale,
                                                          const c10::optional<torch::Tensor>& activation_scale,
                                                          const c10::optional<torch::Tensor>& quant_scale,
                                                          bool activate_left)
{
    const c10::cuda::OptionalCUDAGuard guard(x.device());
    TORCH_CHECK(x.dim() == 2, "dequant_swiglu_quant requires a 2D input [TokensNum, 2H].");
    TORCH_CHECK(x.is_contiguous(), "dequant_swiglu_quant requires a contiguous input.");
    auto outs = dqsq_meta(x, weight_scale, activation_scale, quant_scale, activate_left);
    const int64_t M = x.size(0), N2 = x.size(1);
    if (M <= 0 || N2 <= 0) {
        return outs;
    }
    const int64_t H = N2 / 2;
    const auto xt = x.scalar_type();
    const bool is_i32 = (xt == torch::kInt);
    if (is_i32) {
        TORCH_CHECK(present(weight_scale), "weight_scale is required when x is int32.");
        TORCH_CHECK(present(activation_scale), "activation_scale is required when x is int32.");
        TORCH_CHECK(weight_scale->scalar_type() == torch::kFloat, "weight_scale must be float32.");
        TORCH_CHECK(activation_scale->scalar_type() == torch::kFloat, "activation_scale must be float32.");
        TORCH_CHECK(weight_scale->is_contiguous() && activation_scale->is_contiguous(),
                    "weight_scale / activation_scale must be contiguous.");
        TORCH_CHECK(weight_scale->numel() == N2, "weight_scale must have 2H elements.");
        TORCH_CHECK(activation_scale->numel() == M, "activation_scale must have TokensNum elements.");
    } else {
        TORCH_CHECK(xt == torch::kFloat16 || xt == torch::kBFloat16,
                    "dequant_swiglu_quant supports int32 / float16 / bfloat16 inputs.");
        TORCH_CHECK(!present(weight_scale), "weight_scale must be None for float16 / bfloat16 inputs.");
        TORCH_CHECK(!present(activation_scale), "activation_scale must be None for float16 / bfloat16 inputs.");
    }
    const bool has_q = present(quant_scale);
    if (has_q) {
        TORCH_CHECK(quant_scale->scalar_type() == torch::kFloat, "quant_scale must be float32.");
        TORCH_CHECK(quant_scale->is_contiguous(), "quant_scale must be contiguous.");
        TORCH_CHECK(quant_scale->numel() == H, "quant_scale must have H elements.");
    }
    const int code = is_i32 ? W8A8_DT_I32 : dtype_code(x);
    check_status(w8a8_dequant_swiglu_quant(x.data_ptr(),
                                           is_i32 ? static_cast<const float*>(weight_scale->data_ptr()) : nullptr,
                                           is_i32 ? static_cast<const float*>(activation_scale->data_ptr()) : nullptr,
                                           has_q ? static_cast<const float*>(quant_scale->data_ptr()) : nullptr,
                                           static_cast<int8_t*>(std::get<0>(outs).data_ptr()),
                                           static_cast<float*>(std::get<1>(outs).data_ptr()), M, H, code,
                                           activate_left ? 1 : 0, 0, stream_of(x)),
                 "dequant_swiglu_quant");
    return outs;
}

TORCH_LIBRARY_FRAGMENT(cann_bench, m)
{
    m.def("dequant_swiglu_quant(Tensor x, Tensor? weight_scale=None, Tensor? activation_scale=None, "
          "Tensor? quant_scale=None, bool activate_left=False) -> (Tensor y, Tensor scale)");
    m.def("moe_gating_top_k_softmax(Tensor x, Tensor? finished=None, int k=1) -> "
          "(Tensor y, Tensor expert_idx, Tensor row_idx)");
    m.def("moe_finalize_routing(Tensor expanded_permuted_rows, Tensor expanded_src_to_dst_row, "
          "Tensor? skip1=None, Tensor? skip2=None, Tensor? bias=None, Tensor? scales=None, "
          "Tensor? expert_for_source_row=None, int drop_pad_mode=0) -> Tensor out");
    m.def("moe_re_routing(Tensor tokens, Tensor expert_token_num_per_rank, Tensor? per_token_scales=None, "
          "int expert_token_num_type=1, int idx_type=0) -> (Tensor, Tensor, Tensor, Tensor)");
    m.def("dynamic_quant(Tensor x) -> (Tensor y, Tensor scale)");
    m.def("add_rms_norm_dynamic_quant(Tensor x1, Tensor x2, Tensor gamma, float epsilon) -> "
          "(Tensor y, Tensor xOut, Tensor scaleOut)");
    m.def("quant_matmul(Tensor x1, Tensor x2, Tensor scale, *, Tensor? offset=None, "
          "Tensor? pertoken_scale=None, Tensor? bias=None, str? output_dtype=None) -> Tensor");
    m.def("grouped_matmul_swiglu_quant(Tensor x, Tensor weight, Tensor weight_scale, Tensor x_scale, "
          "int[] group_list) -> (Tensor y, Tensor y_scale)");
    // the two trailing optional scales are this build's extension for the int8 down projection;
    // omitted, the schema and behaviour are the reference's
    m.def("grouped_matmul(Tensor x, Tensor weight, int[] group_list, Tensor? bias=None, int split_item=0, "
          "bool transpose_weight=False, Tensor? x_scale=None, Tensor? weight_scale=None) -> Tensor[]");
}

TORCH_LIBRARY_IMPL(cann_bench, Meta, m)
{
    m.impl("dynamic_quant", dynamic_quant_meta);
    m.impl("add_rms_norm_dynamic_quant", ardq_meta);
    m.impl("quant_matmul", quant_matmul_meta);
    m.impl("grouped_matmul_swiglu_quant", gmsq_meta);
    m.impl("grouped_matmul", grouped_matmul_meta);
    m.impl("moe_re_routing", moe_re_routing_meta);
    m.impl("moe_finalize_routing", mfr_meta);
    m.impl("moe_gating_top_k_softmax", gating_meta);
    m.impl("dequant_swiglu_quant", dqsq_meta);
}

TORCH_LIBRARY_IMPL(cann_bench, CUDA, m)
{
    m.impl("dynamic_quant", dynamic_quant_cuda);
    m.impl("add_rms_norm_dynamic_quant", ardq_cuda);
    m.impl("quant_matmul", quant_matmul_cuda);
    m.impl("grouped_matmul_swiglu_quant", gmsq_cuda);
    m.impl("grouped_matmul", grouped_matmul_cuda);
    m.impl("moe_re_routing", moe_re_routing_cuda);
    m.impl("moe_finalize_routing", mfr_cuda);
    m.impl("moe_gating_top_k_softmax", gating_cuda);
    m.impl("dequant_swiglu_quant", dqsq_cuda);
}

}  // namespace cann_bench
