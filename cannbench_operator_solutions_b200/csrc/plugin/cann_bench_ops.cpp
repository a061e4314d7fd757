// torch operator plugin: registers the operator schemas of the catalog's W8A8
// FFN path in namespace cann_bench and implements them for the CUDA dispatch
// key on top of the C-ABI in include/w8a8ffn.h.
//
// The schema strings are the reference's (they are the interface callers bind
// to):
//   dynamic_quant               operators/dynamicquant/csrc/ops/dynamic_quant/op_plugin/dynamic_quant_plugin.cpp:30
//   add_rms_norm_dynamic_quant  operators/addrmsnormdynamicquant/csrc/ops/add_rms_norm_dynamic_quant/op_plugin/add_rms_norm_dynamic_quant_plugin.cpp:32
//   quant_matmul                operators/quantmatmul/csrc/ops/quant_matmul/op_plugin/quant_matmul_plugin.cpp:48-49
//   grouped_matmul_swiglu_quant operators/groupedmatmulswigluquant/csrc/ops/grouped_matmul_swiglu_quant/op_plugin/gmsq_plugin.cpp:40-41
//   grouped_matmul              operators/groupedmatmul/csrc/ops/grouped_matmul/op_plugin/grouped_matmul_plugin.cpp:42-43
//   moe_re_routing              operators/moererouting/csrc/ops/moe_re_routing/op_plugin/moe_re_routing_plugin.cpp:35-38
//   dequant_swiglu_quant        operators/dequantswigluquant/csrc/ops/dequant_swiglu_quant/op_plugin/dqsq_plugin.cpp:34-35
//   moe_gating_top_k_softmax    operators/moegatingtopksoftmax/csrc/ops/moe_gating_top_k_softmax/op_plugin/moe_gating_plugin.cpp:30
//   moe_finalize_routing        operators/moefinalizerouting/csrc/ops/moe_finalize_routing/op_plugin/moe_finalize_routing_plugin.cpp:33-35
//
// Everything below the schemas is organised differently from those plugins.
// Each operator is one struct with two members: `shape()` derives the output
// tensors from the argument shapes alone (it is the Meta implementation), and
// `run()` is the CUDA implementation: it declares every tensor argument to a
// `Call` object - accepted element types, rank range, element count - which
// checks them in one place, makes dense copies where needed and keeps them
// alive, then makes exactly one C-ABI call on the current CUDA stream.  The
// library re-validates sizes and alignment; the plugin only translates torch
// types.  All arithmetic is in the library.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <algorithm>
#include <string>
#include <tuple>
#include <vector>

#include "../../../include/w8a8ffn.h"

namespace cann_bench {
namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

// element types as a bit set, so that an argument's accepted types are one constant
enum TypeBit : unsigned { F16 = 1u, BF16 = 2u, F32 = 4u, I8 = 8u, I32 = 16u, I64 = 32u, BOOL = 64u };
constexpr unsigned HALVES = F16 | BF16;
constexpr unsigned FLOATS = F16 | BF16 | F32;

struct TypeInfo {
    c10::ScalarType torch_type;
    unsigned bit;
    int abi_code;  // W8A8_DT_* or -1
};
constexpr TypeInfo TYPE_TABLE[] = {
    {torch::kFloat16, F16, W8A8_DT_F16}, {torch::kBFloat16, BF16, W8A8_DT_BF16}, {torch::kFloat32, F32, W8A8_DT_F32},
    {torch::kChar, I8, W8A8_DT_I8},      {torch::kInt, I32, W8A8_DT_I32},        {torch::kLong, I64, -1},
    {torch::kBool, BOOL, -1},
};

const TypeInfo* type_info(c10::ScalarType t)
{
    for (const TypeInfo& e : TYPE_TABLE) {
        if (e.torch_type == t) {
            return &e;
        }
    }
    return nullptr;
}

unsigned type_bit(const Tensor& t)
{
    const TypeInfo* e = type_info(t.scalar_type());
    return e != nullptr ? e->bit : 0u;
}

int abi_type(const Tensor& t)
{
    const TypeInfo* e = type_info(t.scalar_type());
    TORCH_CHECK(e != nullptr && e->abi_code >= 0, "unsupported dtype ", t.scalar_type());
    return e->abi_code;
}

bool given(const OptTensor& t) { return t.has_value() && t->defined(); }

std::vector<int64_t> all_but_last(const Tensor& t)
{
    return std::vector<int64_t>(t.sizes().begin(), t.sizes().end() - 1);
}

// The shape functions (the Meta implementations) state their rules with the same vocabulary as Call::in: a rank
// range (hi < 0: no upper bound) and a set of element types per argument.
void rank_between(const Tensor& t, int lo, int hi, const char* message)
{
    TORCH_CHECK(t.dim() >= lo && (hi < 0 || t.dim() <= hi), message);
}
void type_among(const Tensor& t, unsigned types, const char* message)
{
    TORCH_CHECK((type_bit(t) & types) != 0u, message);
}

// One operator invocation: device guard, stream, argument intake, status translation.
class Call {
public:
    Call(const char* op, const Tensor& anchor)
        : op_(op), guard_(anchor.device()),
          stream_(static_cast<void*>(at::cuda::getCurrentCUDAStream(anchor.device().index()).stream()))
    {
    }

    // the message is the whole sentence the user sees; nothing is prefixed, so texts stay greppable
    template <typename... Parts>
    void require(bool ok, const Parts&... parts) const
    {
        TORCH_CHECK(ok, parts...);
    }

    // A mandatory tensor: element type in `types`, rank in [rank_lo, rank_hi] (rank_hi < 0: no upper bound).
    // `dense` asks for a contiguous copy when the tensor is strided; otherwise a strided tensor is an error.
    Tensor in(const Tensor& t, unsigned types, int rank_lo, int rank_hi, const char* type_msg, const char* rank_msg,
              bool dense = true)
    {
        require((type_bit(t) & types) != 0u, type_msg);
        require(t.dim() >= rank_lo && (rank_hi < 0 || t.dim() <= rank_hi), rank_msg);
        if (t.is_contiguous()) {
            return t;
        }
        require(dense, op_, " requires contiguous inputs.");
        held_.push_back(t.contiguous());
        return held_.back();
    }

    // An optional tensor: an undefined Tensor when absent.
    Tensor opt(const OptTensor& t, unsigned types, const char* type_msg, bool dense = true)
    {
        if (!given(t)) {
            return Tensor();
        }
        return in(*t, types, 0, -1, type_msg, type_msg, dense);
    }

    static const void* ptr(const Tensor& t) { return t.defined() ? t.data_ptr() : nullptr; }
    template <typename T>
    static T* as(const Tensor& t)
    {
        return t.defined() ? static_cast<T*>(t.data_ptr()) : nullptr;
    }

    Tensor scratch(size_t bytes, const Tensor& like)
    {
        held_.push_back(torch::empty({static_cast<int64_t>(bytes)}, like.options().dtype(torch::kUInt8)));
        return held_.back();
    }

    void* stream() const { return stream_; }

    void done(int status) const
    {
        TORCH_CHECK(status == W8A8_OK, op_, ": ", w8a8_status_string(status), " (status ", status, ")");
    }

private:
    const char* op_;
    c10::cuda::OptionalCUDAGuard guard_;
    void* stream_;
    std::vector<Tensor> held_;
};

// The cumulative group list as the library takes it (host int64 array), with the checks whose failures a
// Python caller should see as a torch error rather than as a status code.
std::vector<int64_t> group_ends(const c10::List<int64_t>& list, int64_t experts, int64_t rows, const char* op)
{
    TORCH_CHECK(static_cast<int64_t>(list.size()) == experts, op, ": group_list length must equal the expert count");
    std::vector<int64_t> ends;
    ends.reserve(static_cast<size_t>(experts));
    int64_t floor = 0;
    bool sorted = true;
    for (size_t i = 0; i < list.size(); ++i) {
        const int64_t v = list.get(i);
        sorted = sorted && v >= floor && v <= rows;
        floor = v;
        ends.push_back(v);
    }
    TORCH_CHECK(sorted, op, ": group_list must be a cumsum <= M");
    TORCH_CHECK(floor == rows, op, ": group_list[-1] must equal M");
    return ends;
}

// The tensor-core kernels take K in multiples of 16 bytes (8 elements for 16- and 32-bit operands) and N in multiples
// of 16; the schemas accept any K and N.  Shapes in between are run on zero-padded copies and the result is cut
// back: a zero K column adds nothing to any accumulator, and padded N columns are never returned, so the
// returned elements are those of the unpadded problem bit for bit.
int64_t round_up(int64_t v, int64_t to) { return (v + to - 1) / to * to; }

// `t` with its last dimension zero-padded from its present size to `size` (the tensor itself when nothing is to add)
Tensor widen_last(const Tensor& t, int64_t size)
{
    if (!t.defined() || t.size(-1) == size) {
        return t;
    }
    return torch::constant_pad_nd(t, {0, size - t.size(-1)}, 0).contiguous();
}

// the last two dimensions zero-padded to [rows, cols]
Tensor widen_last2(const Tensor& t, int64_t rows, int64_t cols)
{
    if (t.size(-2) == rows && t.size(-1) == cols) {
        return t;
    }
    return torch::constant_pad_nd(t, {0, cols - t.size(-1), 0, rows - t.size(-2)}, 0).contiguous();
}

// ================================================================ dynamic_quant
struct DynamicQuant {
    using Out = std::tuple<Tensor, Tensor>;

    static Out shape(const Tensor& x)
    {
        rank_between(x, 2, -1, "dynamic_quant requires a tensor with rank >= 2.");
        type_among(x, HALVES, "dynamic_quant only supports float16 / bfloat16 inputs.");
        return {torch::empty_like(x, x.options().dtype(torch::kChar)),
                torch::empty(all_but_last(x), x.options().dtype(torch::kFloat))};
    }

    static Out run(const Tensor& x)
    {
        Call call("dynamic_quant", x);
        const Tensor xd = call.in(x, HALVES, 2, -1, "dynamic_quant only supports float16 / bfloat16 inputs.",
                                  "dynamic_quant requires a tensor with rank >= 2.");
        Out out = shape(xd);
        const int64_t width = xd.size(-1);
        call.require(width > 0, "dynamic_quant requires a non-zero last dimension.");
        if (xd.numel() > 0) {
            call.done(w8a8_dynamic_quant(xd.data_ptr(), Call::as<int8_t>(std::get<0>(out)),
                                         Call::as<float>(std::get<1>(out)), xd.numel() / width, width, abi_type(xd),
                                         0, call.stream()));
        }
        return out;
    }
};

// =================================================== add_rms_norm_dynamic_quant
struct AddRmsNormDynamicQuant {
    using Out = std::tuple<Tensor, Tensor, Tensor>;

    static Out shape(const Tensor& x1, const Tensor& x2, const Tensor& gamma, double /*epsilon*/)
    {
        rank_between(x1, 1, -1, "add_rms_norm_dynamic_quant: x1 must have at least one dimension.");
        TORCH_CHECK(x2.sizes().equals(x1.sizes()), "add_rms_norm_dynamic_quant: x1 and x2 must share a shape.");
        const char* gamma_shape = "add_rms_norm_dynamic_quant: gamma must be 1-D with size == x1.size(-1).";
        rank_between(gamma, 1, 1, gamma_shape);
        TORCH_CHECK(gamma.size(0) == x1.size(-1), gamma_shape);
        type_among(gamma, type_bit(x1), "add_rms_norm_dynamic_quant: gamma dtype must match x1 dtype.");
        return {torch::empty_like(x1, x1.options().dtype(torch::kChar)), torch::empty_like(x1),
                torch::empty(all_but_last(x1), x1.options().dtype(torch::kFloat))};
    }

    static Out run(const Tensor& x1, const Tensor& x2, const Tensor& gamma, double epsilon)
    {
        Call call("add_rms_norm_dynamic_quant", x1);
        if (x1.numel() == 0) {
            return shape(x1, x2, gamma, epsilon);
        }
        const char* types = "add_rms_norm_dynamic_quant: only float16/bfloat16 inputs are supported.";
        const char* rank = "add_rms_norm_dynamic_quant: x1 must have at least one dimension.";
        const Tensor a = call.in(x1, HALVES, 1, -1, types, rank);
        const Tensor b = call.in(x2, type_bit(a), 1, -1, "add_rms_norm_dynamic_quant: x2 dtype must match x1 dtype.",
                                 rank);
        const Tensor g = call.in(gamma, type_bit(a), 1, 1, "add_rms_norm_dynamic_quant: gamma dtype must match x1 dtype.",
                                 "add_rms_norm_dynamic_quant: gamma must be 1-D with size == x1.size(-1).");
        const int64_t width = a.size(-1);
        call.require(width <= 16384, "add_rms_norm_dynamic_quant: row length must not exceed 16384.");
        Out out = shape(a, b, g, epsilon);  // shaped like the dense copies: the library writes dense rows
        call.done(w8a8_add_rms_norm_dynamic_quant(a.data_ptr(), b.data_ptr(), g.data_ptr(),
                                                  Call::as<int8_t>(std::get<0>(out)), std::get<1>(out).data_ptr(),
                                                  Call::as<float>(std::get<2>(out)),
                                                  a.numel() / width, width, static_cast<float>(epsilon), abi_type(a),
                                                  0, call.stream()));
        return out;
    }
};

// ================================================================= quant_matmul
struct QuantMatmul {
    static Tensor shape(const Tensor& x1, const Tensor& x2, const Tensor& /*scale*/, const OptTensor& /*offset*/,
                        const OptTensor& /*pertoken_scale*/, const OptTensor& /*bias*/,
                        const c10::optional<std::string>& output_dtype)
    {
        rank_between(x1, 2, -1, "quant_matmul requires inputs of rank >= 2.");
        rank_between(x2, 2, -1, "quant_matmul requires inputs of rank >= 2.");
        TORCH_CHECK(x2.size(-2) == x1.size(-1), "quant_matmul requires x1.size(-1) == x2.size(-2).");
        std::vector<int64_t> dims = all_but_last(x1);
        dims.push_back(x2.size(-1));
        const bool bf16 = output_dtype.has_value() && *output_dtype == "bfloat16";
        return torch::empty(dims, x1.options().dtype(bf16 ? torch::kBFloat16 : torch::kFloat16));
    }

    // One per-channel-or-scalar operand of the epilogue: which flag bits it raises.
    struct Term {
        const Tensor* t;
        int64_t present;
        int64_t per_channel;
        const char* size_msg;
    };

    static Tensor run(const Tensor& x1, const Tensor& x2, const Tensor& scale, const OptTensor& offset,
                      const OptTensor& pertoken_scale, const OptTensor& bias,
                      const c10::optional<std::string>& output_dtype)
    {
        Call call("quant_matmul", x1);
        const char* i8 = "quant_matmul requires int8 x1 and x2.";
        const char* rk = "quant_matmul expects equal ranks >= 2.";
        const Tensor a = call.in(x1, I8, 2, -1, i8, rk, /*dense=*/false);
        const Tensor b = call.in(x2, I8, static_cast<int>(x1.dim()), static_cast<int>(x1.dim()), i8, rk, false);
        const Tensor sc = call.in(scale, F32 | BF16, 0, -1, "quant_matmul requires float32 or bfloat16 scale.", rk, false);
        const Tensor off = call.opt(offset, F32, "quant_matmul requires float32 contiguous offset.", false);
        const Tensor pt = call.opt(pertoken_scale, F32, "quant_matmul requires float32 contiguous pertoken_scale.", false);
        const Tensor bs = call.opt(bias, I32 | FLOATS, "quant_matmul unsupported bias dtype", false);
        Tensor out = shape(a, b, sc, offset, pertoken_scale, bias, output_dtype);

        const int64_t rows = a.size(-2), depth = a.size(-1), cols = b.size(-1);
        call.require(rows > 0 && depth > 0 && cols > 0, "quant_matmul requires non-empty shapes.");
        call.require(a.sizes().slice(0, a.dim() - 2) == b.sizes().slice(0, b.dim() - 2),
                     "quant_matmul expects matching leading batch dimensions.");
        const int64_t batch = a.numel() / (rows * depth);

        // a bias shaped [batch, 1, cols] carries one row per batch entry; anything else is shared by all of them
        const bool bias_per_batch = bs.defined() && batch > 1 && bs.dim() == 3 && bs.size(0) == batch &&
                                    bs.size(1) == 1 && bs.size(2) == cols;
        int64_t flags = (batch > 1) ? W8A8_QM_PT_MOD_M : 0;
        const Term terms[] = {
            {&sc, 0, W8A8_QM_SCALE_PERCHAN, "quant_matmul expects scale length 1 or n."},
            {&off, W8A8_QM_HAS_OFFSET, W8A8_QM_OFFSET_PERCHAN, "quant_matmul expects offset length 1 or n."},
            {&bs, 0, W8A8_QM_BIAS_PERCHAN, "quant_matmul expects bias length 1 or n."},
        };
        for (const Term& term : terms) {
            if (!term.t->defined()) {
                continue;
            }
            const int64_t count = (term.t == &bs && bias_per_batch) ? cols : term.t->numel();
            call.require(count == 1 || count == cols, term.size_msg);
            flags |= term.present | (count > 1 ? term.per_channel : 0);
        }
        if (sc.scalar_type() == torch::kBFloat16) {
            flags |= W8A8_QM_SCALE_BF16;
        }
        if (pt.defined()) {
            call.require(pt.numel() == rows, "quant_matmul expects pertoken_scale length m.");
            flags |= W8A8_QM_HAS_PT;
        }
        if (bs.defined()) {
            constexpr struct {
                unsigned bit;
                int64_t kind;
            } kinds[] = {{I32, W8A8_QM_BIAS_I32}, {F16, W8A8_QM_BIAS_F16}, {BF16, W8A8_QM_BIAS_BF16},
                         {F32, W8A8_QM_BIAS_F32}};
            for (const auto& k : kinds) {
                if (type_bit(bs) == k.bit) {
                    flags |= k.kind << W8A8_QM_BIAS_SHIFT;
                }
            }
        }
        // K and N as the kernels take them; per-channel operands grow with N (a scalar stays a scalar)
        const int64_t depth_p = round_up(depth, 16), cols_p = round_up(cols, 16);
        const bool padded = depth_p != depth || cols_p != cols;
        const auto per_channel = [&](const Tensor& t) {
            return (t.defined() && t.numel() > 1) ? widen_last(t.reshape({-1, cols}), cols_p) : t;
        };
        const Tensor a_p = widen_last(a, depth_p), b_p = widen_last2(b, depth_p, cols_p);
        const Tensor sc_p = per_channel(sc), off_p = per_channel(off), bs_p = per_channel(bs);
        Tensor out_p = out;
        if (padded) {
            std::vector<int64_t> dims = all_but_last(out);
            dims.push_back(cols_p);
            out_p = torch::empty(dims, out.options());
        }
        call.done(w8a8_quant_matmul(Call::as<const int8_t>(a_p), Call::as<const int8_t>(b_p), sc_p.data_ptr(),
                                    Call::as<const float>(off_p), Call::as<const float>(pt), Call::ptr(bs_p),
                                    out_p.data_ptr(), batch, rows, cols_p, depth_p, flags,
                                    out.scalar_type() == torch::kBFloat16 ? W8A8_DT_BF16 : W8A8_DT_F16, W8A8_W_KN,
                                    bias_per_batch ? cols_p : 0, call.stream()));
        if (padded) {
            out.copy_(out_p.narrow(-1, 0, cols));
        }
        return out;
    }
};

// ================================================== grouped_matmul_swiglu_quant
struct GroupedMatmulSwigluQuant {
    using Out = std::tuple<Tensor, Tensor>;

    static Out shape(const Tensor& x, const Tensor& weight, const Tensor& /*weight_scale*/, const Tensor& /*x_scale*/,
                     c10::List<int64_t> /*group_list*/)
    {
        rank_between(x, 2, 2, "grouped_matmul_swiglu_quant: x must be 2D [M, K]");
        rank_between(weight, 3, 3, "grouped_matmul_swiglu_quant: weight must be 3D [E, K, N]");
        TORCH_CHECK(weight.size(2) % 2 == 0, "grouped_matmul_swiglu_quant: N must be even");
        return {torch::empty({x.size(0), weight.size(2) / 2}, x.options().dtype(torch::kChar)),
                torch::empty({x.size(0)}, x.options().dtype(torch::kFloat32))};
    }

    static Out run(const Tensor& x, const Tensor& weight, const Tensor& weight_scale, const Tensor& x_scale,
                   c10::List<int64_t> group_list)
    {
        Call call("grouped_matmul_swiglu_quant", x);
        const Tensor rows = call.in(x, I8, 2, 2, "grouped_matmul_swiglu_quant: x must be int8",
                                    "grouped_matmul_swiglu_quant: x must be 2D [M, K]");
        const Tensor w = call.in(weight, I8, 3, 3, "grouped_matmul_swiglu_quant: weight must be int8",
                                 "grouped_matmul_swiglu_quant: weight must be 3D [E, K, N]");
        const Tensor ws = call.in(weight_scale, F32, 0, -1, "grouped_matmul_swiglu_quant: weight_scale must be float32",
                                  "grouped_matmul_swiglu_quant: weight_scale must be [E, N]");
        const Tensor xs = call.in(x_scale, F32, 0, -1, "grouped_matmul_swiglu_quant: x_scale must be float32",
                                  "grouped_matmul_swiglu_quant: x_scale must have M elements");
        Out out = shape(rows, w, ws, xs, group_list);
        const int64_t m = rows.size(0), k = rows.size(1), e = w.size(0), n = w.size(2);
        if (m == 0 || n == 0 || e == 0) {
            return out;
        }
        call.require(w.size(1) == k, "grouped_matmul_swiglu_quant: K mismatch between x and weight");
        call.require(xs.numel() == m, "grouped_matmul_swiglu_quant: x_scale must have M elements");
        call.require(ws.dim() == 2 && ws.size(0) == e && ws.size(1) == n,
                     "grouped_matmul_swiglu_quant: weight_scale must be [E, N]");
        const std::vector<int64_t> ends = group_ends(group_list, e, m, "grouped_matmul_swiglu_quant");
        // The gate columns are the first half of N and the up columns the second: each half is padded on its own.
        // A padded column has weight 0, so its activation is silu(0) * 0 = 0: it neither moves the row maximum
        // nor is it returned.
        const int64_t half = n / 2, half_p = round_up(half, 16), k_p = round_up(k, 16);
        const bool padded = half_p != half || k_p != k;
        Tensor rows_p = rows, w_p = w, ws_p = ws, y_p = std::get<0>(out);
        if (padded) {
            rows_p = widen_last(rows, k_p);
            w_p = torch::cat({widen_last2(w.narrow(2, 0, half), k_p, half_p), widen_last2(w.narrow(2, half, half), k_p, half_p)},
                             2)
                      .contiguous();
            ws_p = torch::cat({widen_last(ws.narrow(1, 0, half), half_p), widen_last(ws.narrow(1, half, half), half_p)}, 1)
                       .contiguous();
            y_p = torch::empty({m, half_p}, y_p.options());
        }
        const size_t bytes = w8a8_grouped_matmul_swiglu_quant_workspace_size(m, k_p, 2 * half_p, e);
        const Tensor ws_buf = call.scratch(bytes, rows);
        call.done(w8a8_grouped_matmul_swiglu_quant(Call::as<const int8_t>(rows_p), Call::as<const int8_t>(w_p),
                                                   Call::as<const float>(ws_p), Call::as<const float>(xs),
                                                   Call::as<int8_t>(y_p), Call::as<float>(std::get<1>(out)), m, k_p,
                                                   2 * half_p, e, ends.data(), 0, W8A8_W_KN, 0, ws_buf.data_ptr(),
                                                   bytes, call.stream()));
        if (padded) {
            std::get<0>(out).copy_(y_p.narrow(1, 0, half));
        }
        return out;
    }
};

// =============================================================== grouped_matmul
struct GroupedMatmul {
    using Out = c10::List<Tensor>;

    // split_item 0 / 1: one view of the joined result per expert; 2 / 3: the joined result alone
    static Out views(const Tensor& joined, const std::vector<int64_t>& ends, int64_t split_item)
    {
        Out list;
        if (split_item >= 2) {
            list.push_back(joined);
            return list;
        }
        int64_t begin = 0;
        for (const int64_t end : ends) {
            list.push_back(joined.narrow(0, begin, end - begin));
            begin = end;
        }
        return list;
    }

    static Tensor joined(const Tensor& x, const Tensor& weight, bool transpose_weight, const OptTensor& x_scale)
    {
        rank_between(x, 2, 2, "grouped_matmul: x must be 2D [M, K]");
        rank_between(weight, 3, 3, "grouped_matmul: weight must be 3D [E, K, N] or [E, N, K]");
        const int64_t n = weight.size(transpose_weight ? 1 : 2);
        // the quantised form (this build's extension) always answers in bfloat16
        return torch::empty({x.size(0), n}, given(x_scale) ? x.options().dtype(torch::kBFloat16) : x.options());
    }

    static Out shape(const Tensor& x, const Tensor& weight, c10::List<int64_t> group_list, const OptTensor& /*bias*/,
                     int64_t split_item, bool transpose_weight, const OptTensor& x_scale,
                     const OptTensor& /*weight_scale*/)
    {
        const Tensor y = joined(x, weight, transpose_weight, x_scale);
        return views(y, group_ends(group_list, weight.size(0), x.size(0), "grouped_matmul"), split_item);
    }

    static Out run(const Tensor& x, const Tensor& weight, c10::List<int64_t> group_list, const OptTensor& bias,
                   int64_t split_item, bool transpose_weight, const OptTensor& x_scale, const OptTensor& weight_scale)
    {
        Call call("grouped_matmul", x);
        const char* types = "grouped_matmul: x must be float16, bfloat16, float32 or int8";
        const Tensor rows = call.in(x, FLOATS | I8, 2, 2, types, "grouped_matmul: x must be 2D [M, K]");
        const Tensor w = call.in(weight, type_bit(rows), 3, 3, "grouped_matmul: x and weight must share a dtype",
                                 "grouped_matmul: weight must be 3D [E, K, N] or [E, N, K]");
        const bool quantised = type_bit(rows) == I8;
        const int64_t m = rows.size(0), k = rows.size(1), e = w.size(0);
        const int64_t n = w.size(transpose_weight ? 1 : 2);
        call.require(e >= 1, "grouped_matmul: weight must contain at least one expert");
        call.require(w.size(transpose_weight ? 2 : 1) == k, "grouped_matmul: K dimension mismatch between x and weight");
        const std::vector<int64_t> ends = group_ends(group_list, e, m, "grouped_matmul");
        call.require(quantised == given(x_scale) && quantised == given(weight_scale),
                     quantised ? "grouped_matmul: int8 inputs need x_scale and weight_scale"
                               : "grouped_matmul: scales are only valid with int8 inputs");
        const Tensor xs = call.opt(x_scale, F32, "grouped_matmul: x_scale must be fp32 [M]");
        const Tensor ws = call.opt(weight_scale, F32, "grouped_matmul: weight_scale must be fp32 [E, N]");
        call.require(!xs.defined() || xs.numel() == m, "grouped_matmul: x_scale must be fp32 [M]");
        call.require(!ws.defined() || ws.numel() == e * n, "grouped_matmul: weight_scale must be fp32 [E, N]");
        const Tensor b = call.opt(bias, FLOATS, "grouped_matmul: bias must be float16, bfloat16 or float32");
        call.require(!b.defined() || b.numel() == e * n, "grouped_matmul: bias must have shape [E, N]");
        const Tensor y = joined(rows, w, transpose_weight, x_scale);
        if (m > 0) {
            const int64_t k_p = round_up(k, quantised ? 16 : 8), n_p = round_up(n, 16);
            const bool padded = k_p != k || n_p != n;
            Tensor rows_p = rows, w_p = w, b_p = b, ws_p = ws, y_p = y;
            if (padded) {
                rows_p = widen_last(rows, k_p);
                w_p = transpose_weight ? widen_last2(w, n_p, k_p) : widen_last2(w, k_p, n_p);
                b_p = b.defined() ? widen_last(b.reshape({e, n}), n_p) : b;
                ws_p = ws.defined() ? widen_last(ws.reshape({e, n}), n_p) : ws;
                y_p = torch::empty({m, n_p}, y.options());
            }
            const size_t bytes = (type_bit(rows) == F32) ? w8a8_grouped_matmul_f32_workspace_size(m, n_p, k_p, e)
                                                         : w8a8_grouped_matmul_workspace_size(m, n_p, k_p, e);
            const Tensor ws_buf = call.scratch(bytes, rows);
            call.done(w8a8_grouped_matmul(rows_p.data_ptr(), w_p.data_ptr(), Call::ptr(b_p), y_p.data_ptr(),
                                          Call::as<const float>(xs), Call::as<const float>(ws_p), m, n_p, k_p, e,
                                          ends.data(), 0, abi_type(rows), b.defined() ? abi_type(b) : abi_type(rows),
                                          abi_type(y), transpose_weight ? W8A8_W_NK : W8A8_W_KN, ws_buf.data_ptr(),
                                          bytes, call.stream()));
            if (padded) {
                y.copy_(y_p.narrow(1, 0, n));
            }
        }
        return views(y, ends, split_item);
    }
};

// =============================================================== moe_re_routing
struct MoeReRouting {
    using Out = std::tuple<Tensor, Tensor, Tensor, Tensor>;

    static Out shape(const Tensor& tokens, const Tensor& counts, const OptTensor& /*scales*/,
                     int64_t /*expert_token_num_type*/, int64_t /*idx_type*/)
    {
        rank_between(tokens, 2, 2, "moe_re_routing: tokens must be 2D (A, H).");
        rank_between(counts, 2, 2, "moe_re_routing: expert_token_num_per_rank must be 2D (N, E).");
        const int64_t a = tokens.size(0);
        const auto like = tokens.options();
        return {torch::empty({a, tokens.size(1)}, like), torch::empty({a}, like.dtype(torch::kFloat)),
                torch::empty({a}, like.dtype(torch::kInt)), torch::empty({counts.size(1)}, counts.options())};
    }

    static Out run(const Tensor& tokens, const Tensor& counts, const OptTensor& scales, int64_t num_type,
                   int64_t idx_type)
    {
        TORCH_CHECK(idx_type == 0, "moe_re_routing: only gather index mode (idx_type == 0) is supported.");
        Call call("moe_re_routing", tokens);
        Out out = shape(tokens, counts, scales, num_type, idx_type);
        if (tokens.numel() == 0 || counts.numel() == 0) {
            return out;
        }
        const Tensor tok = call.in(tokens, HALVES | I8, 2, 2, "moe_re_routing: unsupported tokens dtype.",
                                   "moe_re_routing: tokens must be 2D (A, H).");
        const Tensor cnt = call.in(counts, I32 | I64, 2, 2, "moe_re_routing: unsupported expert_token_num_per_rank dtype.",
                                   "moe_re_routing: expert_token_num_per_rank must be 2D (N, E).");
        call.require(cnt.is_cuda(), "moe_re_routing: expert_token_num_per_rank must be on the tokens' device.");
        const Tensor scl = call.opt(scales, F32, "moe_re_routing: per_token_scales must be float32.");
        call.require(!scl.defined() || scl.numel() == tok.size(0), "moe_re_routing: per_token_scales must have A elements.");
        const int64_t a = tok.size(0), ranks = cnt.size(0), experts = cnt.size(1);
        const size_t bytes = w8a8_moe_re_routing_workspace_size(a, ranks, experts);
        const Tensor ws_buf = call.scratch(bytes, tok);
        call.done(w8a8_moe_re_routing(tok.data_ptr(), cnt.data_ptr(), Call::as<const float>(scl),
                                      std::get<0>(out).data_ptr(), Call::as<float>(std::get<1>(out)),
                                      Call::as<int32_t>(std::get<2>(out)), std::get<3>(out).data_ptr(), a,
                                      tok.size(1) * static_cast<int64_t>(tok.element_size()), ranks, experts,
                                      static_cast<int>(cnt.element_size()), ws_buf.data_ptr(), bytes, call.stream()));
        return out;
    }
};

// ========================================================= moe_finalize_routing
struct MoeFinalizeRouting {
    struct Dims {
        int64_t tokens, topk, hidden;
    };

    static Dims dims(const Tensor& rows, const Tensor& src_to_dst, const OptTensor& scales)
    {
        rank_between(rows, 2, -1, "moe_finalize_routing: expanded_permuted_rows must have rank >= 2.");
        TORCH_CHECK(src_to_dst.scalar_type() == torch::kInt,
                    "moe_finalize_routing: expanded_src_to_dst_row must be int32.");
        TORCH_CHECK(!given(scales) || scales->dim() == 2, "moe_finalize_routing: scales must be 2-D (NUM_ROWS, K).");
        const int64_t topk = given(scales) ? scales->size(1) : 1;
        TORCH_CHECK(topk > 0, "moe_finalize_routing: K must be positive.");
        TORCH_CHECK(src_to_dst.numel() % topk == 0,
                    "moe_finalize_routing: expanded_src_to_dst_row length must be K*NUM_ROWS.");
        return {src_to_dst.numel() / topk, topk, rows.size(-1)};
    }

    static Tensor shape(const Tensor& rows, const Tensor& src_to_dst, OptTensor /*skip1*/, OptTensor /*skip2*/,
                        OptTensor /*bias*/, OptTensor scales, OptTensor /*expert*/, int64_t /*drop_pad_mode*/)
    {
        const Dims d = dims(rows, src_to_dst, scales);
        return torch::empty({d.tokens, d.hidden}, rows.options());
    }

    static Tensor run(const Tensor& rows, const Tensor& src_to_dst, OptTensor skip1, OptTensor skip2, OptTensor bias,
                      OptTensor scales, OptTensor expert, int64_t drop_pad_mode)
    {
        type_among(rows, FLOATS, "moe_finalize_routing: expanded_permuted_rows must be float16 / float32 / bfloat16.");
        Call call("moe_finalize_routing", rows);
        const Dims d = dims(rows, src_to_dst, scales);
        Tensor out = torch::empty({d.tokens, d.hidden}, rows.options());
        if (d.tokens <= 0 || d.hidden <= 0) {
            return out;
        }
        const unsigned row_type = type_bit(rows);
        const Tensor epr = call.in(rows, FLOATS, 2, -1, "moe_finalize_routing: unsupported rows dtype.",
                                   "moe_finalize_routing: expanded_permuted_rows must have rank >= 2.");
        const Tensor map = call.in(src_to_dst, I32, 0, -1, "moe_finalize_routing: expanded_src_to_dst_row must be int32.",
                                   "moe_finalize_routing: expanded_src_to_dst_row must be int32.");
        const Tensor s1 = call.opt(skip1, row_type, "moe_finalize_routing: skip1 must have the rows' dtype.");
        const Tensor s2 = call.opt(skip2, row_type, "moe_finalize_routing: skip2 must have the rows' dtype.");
        const Tensor sc = call.opt(scales, FLOATS,
                                   "moe_finalize_routing: unsupported dtype combination for expanded_permuted_rows / scales.");
        // the bias rows are selected by expert id: without the ids the bias is not applied
        Tensor bs, ex;
        if (given(bias) && given(expert)) {
            bs = call.opt(bias, row_type, "moe_finalize_routing: bias must have the rows' dtype.");
            ex = call.opt(expert, I32, "moe_finalize_routing: expert_for_source_row must be int32.");
            call.require(bs.dim() == 2 && bs.size(1) == d.hidden, "moe_finalize_routing: bias head dim must equal H.");
        }
        const int mode = static_cast<int>(std::min<int64_t>(3, std::max<int64_t>(0, drop_pad_mode)));
        call.done(w8a8_moe_finalize_routing(epr.data_ptr(), Call::as<const int32_t>(map), Call::ptr(s1), Call::ptr(s2),
                                            Call::ptr(bs), Call::ptr(sc), Call::as<const int32_t>(ex), out.data_ptr(),
                                            d.tokens, d.hidden, d.topk, bs.defined() ? bs.size(0) : 0,
                                            epr.numel() / d.hidden, mode, abi_type(epr),
                                            sc.defined() ? abi_type(sc) : abi_type(epr), call.stream()));
        return out;
    }
};

// ===================================================== moe_gating_top_k_softmax
struct MoeGatingTopKSoftmax {
    using Out = std::tuple<Tensor, Tensor, Tensor>;

    static Out shape(const Tensor& x, const OptTensor& finished, int64_t k)
    {
        type_among(x, FLOATS, "cann_bench.moe_gating_top_k_softmax only supports float32, float16 and bfloat16 inputs.");
        rank_between(x, 2, -1, "cann_bench.moe_gating_top_k_softmax requires a tensor with rank >= 2.");
        TORCH_CHECK(x.size(-1) > 0, "cann_bench.moe_gating_top_k_softmax requires a non-empty last dimension.");
        TORCH_CHECK(k > 0 && k <= x.size(-1), "cann_bench.moe_gating_top_k_softmax requires 0 < k <= x.size(-1).");
        TORCH_CHECK(!given(finished) || finished->scalar_type() == torch::kBool,
                    "cann_bench.moe_gating_top_k_softmax requires a bool 'finished' tensor.");
        std::vector<int64_t> dims = all_but_last(x);
        dims.push_back(k);
        const auto ints = x.options().dtype(torch::kInt);
        return {torch::empty(dims, x.options()), torch::empty(dims, ints), torch::empty(dims, ints)};
    }

    static Out run(const Tensor& x, const OptTensor& finished, int64_t k)
    {
        Call call("moe_gating_top_k_softmax", x);
        Out out = shape(x, finished, k);
        const Tensor logits = call.in(x, FLOATS, 2, -1, "unsupported dtype", "rank");
        const int64_t experts = logits.size(-1), rows = logits.numel() / experts;
        call.require(rows > 0, "cann_bench.moe_gating_top_k_softmax requires at least one row.");
        const Tensor fin = call.opt(finished, BOOL, "cann_bench.moe_gating_top_k_softmax requires a bool 'finished' tensor.");
        call.require(!fin.defined() || fin.numel() == rows,
                     "cann_bench.moe_gating_top_k_softmax: finished must have numel == rows.");
        call.done(w8a8_moe_gating_top_k_softmax(logits.data_ptr(), Call::as<const uint8_t>(fin),
                                                std::get<0>(out).data_ptr(), Call::as<int32_t>(std::get<1>(out)),
                                                Call::as<int32_t>(std::get<2>(out)), rows, experts, k,
                                                abi_type(logits), call.stream()));
        return out;
    }
};

// ========================================================= dequant_swiglu_quant
struct DequantSwigluQuant {
    using Out = std::tuple<Tensor, Tensor>;

    static Out shape(const Tensor& x, const OptTensor& /*weight_scale*/, const OptTensor& /*activation_scale*/,
                     const OptTensor& /*quant_scale*/, bool /*activate_left*/)
    {
        rank_between(x, 2, 2, "dequant_swiglu_quant requires a 2D input [TokensNum, 2H].");
        TORCH_CHECK(x.size(1) % 2 == 0, "dequant_swiglu_quant requires an even last dimension.");
        return {torch::empty({x.size(0), x.size(1) / 2}, x.options().dtype(torch::kChar)),
                torch::empty({x.size(0)}, x.options().dtype(torch::kFloat))};
    }

    static Out run(const Tensor& x, const OptTensor& weight_scale, const OptTensor& activation_scale,
                   const OptTensor& quant_scale, bool activate_left)
    {
        Call call("dequant_swiglu_quant", x);
        Out out = shape(x, weight_scale, activation_scale, quant_scale, activate_left);
        const int64_t tokens = x.size(0), half = x.size(1) / 2;
        if (x.numel() == 0) {
            return out;
        }
        const Tensor acc = call.in(x, I32 | HALVES, 2, 2, "dequant_swiglu_quant supports int32 / float16 / bfloat16 inputs.",
                                   "dequant_swiglu_quant requires a 2D input [TokensNum, 2H].", /*dense=*/false);
        const bool integer = type_bit(acc) == I32;
        // an int32 accumulator needs both dequantisation scales; a float input must come without them
        call.require(integer == given(weight_scale), integer ? "weight_scale is required when x is int32."
                                                             : "weight_scale must be None for float16 / bfloat16 inputs.");
        call.require(integer == given(activation_scale),
                     integer ? "activation_scale is required when x is int32."
                             : "activation_scale must be None for float16 / bfloat16 inputs.");
        const struct {
            const OptTensor* arg;
            int64_t count;
            const char* type_msg;
            const char* size_msg;
        } vectors[] = {
            {&weight_scale, 2 * half, "weight_scale must be float32.", "weight_scale must have 2H elements."},
            {&activation_scale, tokens, "activation_scale must be float32.", "activation_scale must have TokensNum elements."},
            {&quant_scale, half, "quant_scale must be float32.", "quant_scale must have H elements."},
        };
        Tensor dense[3];
        for (int i = 0; i < 3; ++i) {
            dense[i] = call.opt(*vectors[i].arg, F32, vectors[i].type_msg, /*dense=*/false);
            call.require(!dense[i].defined() || dense[i].numel() == vectors[i].count, vectors[i].size_msg);
        }
        call.done(w8a8_dequant_swiglu_quant(acc.data_ptr(), Call::as<const float>(dense[0]),
                                            Call::as<const float>(dense[1]), Call::as<const float>(dense[2]),
                                            Call::as<int8_t>(std::get<0>(out)), Call::as<float>(std::get<1>(out)),
                                            tokens, half, integer ? W8A8_DT_I32 : abi_type(acc), activate_left ? 1 : 0,
                                            0, call.stream()));
        return out;
    }
};

}  // namespace

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
    m.impl("dynamic_quant", DynamicQuant::shape);
    m.impl("add_rms_norm_dynamic_quant", AddRmsNormDynamicQuant::shape);
    m.impl("quant_matmul", QuantMatmul::shape);
    m.impl("grouped_matmul_swiglu_quant", GroupedMatmulSwigluQuant::shape);
    m.impl("grouped_matmul", GroupedMatmul::shape);
    m.impl("moe_re_routing", MoeReRouting::shape);
    m.impl("moe_finalize_routing", MoeFinalizeRouting::shape);
    m.impl("moe_gating_top_k_softmax", MoeGatingTopKSoftmax::shape);
    m.impl("dequant_swiglu_quant", DequantSwigluQuant::shape);
}

TORCH_LIBRARY_IMPL(cann_bench, CUDA, m)
{
    m.impl("dynamic_quant", DynamicQuant::run);
    m.impl("add_rms_norm_dynamic_quant", AddRmsNormDynamicQuant::run);
    m.impl("quant_matmul", QuantMatmul::run);
    m.impl("grouped_matmul_swiglu_quant", GroupedMatmulSwigluQuant::run);
    m.impl("grouped_matmul", GroupedMatmul::run);
    m.impl("moe_re_routing", MoeReRouting::run);
    m.impl("moe_finalize_routing", MoeFinalizeRouting::run);
    m.impl("moe_gating_top_k_softmax", MoeGatingTopKSoftmax::run);
    m.impl("dequant_swiglu_quant", DequantSwigluQuant::run);
}

}  // namespace cann_bench
