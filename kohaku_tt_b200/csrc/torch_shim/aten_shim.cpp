// The aten fused-SDPA overloads on the CUDA key, registered from C++: the counterpart of the
// reference's TORCH_LIBRARY_IMPL block (aten_attention.cpp:959-974; tt_sdpa_overrideable
// :389-713, its backward :715-812, fused_refusal :62-127, tt_fused_sdp_choice :194-219).
//
// A thin shim: it checks the call with the reference's refusal rules, lets torch allocate
// the outputs in the layout each overload's meta kernel promises, fills a
// ktt_b200_attn_args block with raw pointers and element strides and calls the C ABI of
// libktt_b200.so on torch's current stream. Nothing here computes.
//
// Registration is dynamic (ktt_b200_aten_install / _uninstall create and destroy the
// torch::Library object), so that a process can take the overloads out again.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cmath>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>

#include "../../../include/ktt_b200.h"

namespace {

using at::Tensor;

// ---- the kernel scope of the calling thread (kohaku_tt_b200.sdpa_kernel) -------------------
thread_local int g_kernel = KTT_B200_KERNEL_AUTO;   // -1: the scope allows no kernel
thread_local std::string g_scope_names;             // empty outside a scope

// The first condition a call fails, or null (fused_refusal, aten_attention.cpp:62-127, minus
// the rules that only describe Tensix limits).
const char* fused_refusal(const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& mask,
                          double dropout_p, bool is_causal) {
    const bool grads = at::GradMode::is_enabled() && (q.requires_grad() || k.requires_grad() || v.requires_grad());
    for (const Tensor* t : {&q, &k, &v}) {
        const bool ok_dtype = t->scalar_type() == at::kBFloat16 || (t->scalar_type() == at::kFloat && !grads);
        if (t->dim() != 4 || t->numel() == 0 || !ok_dtype || t->scalar_type() != q.scalar_type()) {
            return "q, k and v must be non-empty 4-D bf16 (fp32 without gradients)";
        }
    }
    if (dropout_p != 0.0) return "dropout";
    if (k.size(3) != q.size(3)) return "q and k need one head dim";
    if (k.size(0) != q.size(0) || v.size(0) != q.size(0) || v.size(1) != k.size(1) || q.size(1) % k.size(1) != 0 ||
        v.size(2) != k.size(2)) {
        return "q, k and v shapes do not match (K / V heads must divide Q heads)";
    }
    if (std::max(q.size(3), v.size(3)) > 256) return "head dims above 256 are not taken";
    if (is_causal && mask.has_value() && mask->defined()) return "causal takes no mask";
    if (mask.has_value() && mask->defined()) {
        if (mask->dim() > 4) return "the mask must broadcast to [B, H, Sq, Sk]";
        const int64_t full[4] = {q.size(0), q.size(1), q.size(2), k.size(2)};
        for (int64_t i = 0; i < mask->dim(); ++i) {
            const int64_t s = mask->size(mask->dim() - 1 - i);
            if (s != 1 && s != full[3 - i]) return "the mask must broadcast to [B, H, Sq, Sk]";
        }
    }
    return nullptr;
}

std::string describe(const Tensor& t) {
    std::string s = "[";
    for (int64_t i = 0; i < t.dim(); ++i) s += (i ? ", " : "") + std::to_string(t.size(i));
    return s + "] " + std::string(c10::toString(t.scalar_type()));
}

void checked(const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& mask, double dropout_p,
             bool is_causal) {
    const char* why = fused_refusal(q, k, v, mask, dropout_p, is_causal);
    if (!why) {
        TORCH_CHECK(g_kernel >= 0, "kohaku_tt_b200.sdpa_kernel(", g_scope_names,
                    "): no device kernel is allowed and there is no math fallback");
        return;
    }
    if (!g_scope_names.empty()) {
        std::string m = "none";
        if (mask.has_value() && mask->defined()) m = (mask->scalar_type() == at::kBool ? "bool " : "additive ") + describe(*mask);
        TORCH_CHECK(false, "kohaku_tt_b200.sdpa_kernel(", g_scope_names, "): no allowed kernel takes attention q ", describe(q),
                    ", k ", describe(k), ", v ", describe(v), ", mask ", m, is_causal ? ", causal" : "", ": ", why);
    }
    TORCH_CHECK_NOT_IMPLEMENTED(
        false, "kohaku_tt_b200: fused attention refused: ", why,
        ". On CUDA PyTorch picks the fused overload itself, so a refused call cannot fall back to the math composite from "
        "here: wrap it in torch.nn.attention.sdpa_kernel(SDPBackend.MATH), or call kohaku_tt_b200.uninstall()");
}

void raise_status(int rc, const char* what) {
    if (rc == KTT_B200_OK) return;
    const std::string msg = std::string("kohaku_tt_b200.") + what + ": " + ktt_b200_last_error();
    if (rc == KTT_B200_ERR_UNSUPPORTED) TORCH_CHECK_NOT_IMPLEMENTED(false, msg);
    if (rc == KTT_B200_ERR_BAD_ARGUMENT) TORCH_CHECK_VALUE(false, msg);
    TORCH_CHECK(false, msg);
}

Tensor rows_contiguous(const Tensor& t) { return t.stride(-1) == 1 ? t : t.contiguous(); }

void set3(int64_t* dst, const Tensor& t) {
    dst[0] = t.stride(0);
    dst[1] = t.stride(1);
    dst[2] = t.stride(2);
}

// Mask operand: expanded view (kept alive by the caller through `keep`), dtype code, strides.
void mask_operand(ktt_b200_attn_args& a, const c10::optional<Tensor>& mask, int64_t b, int64_t h, int64_t sq, int64_t sk, Tensor& keep) {
    a.mask = nullptr;
    a.mask_dtype = KTT_B200_MASK_NONE;
    if (!mask.has_value() || !mask->defined()) return;
    Tensor m = *mask;
    int code;
    switch (m.scalar_type()) {
        case at::kBool: case at::kByte: code = KTT_B200_MASK_BOOL; break;
        case at::kBFloat16: code = KTT_B200_MASK_BF16; break;
        case at::kFloat: code = KTT_B200_MASK_F32; break;
        case at::kHalf: code = KTT_B200_MASK_F16; break;
        default: m = m.to(at::kFloat); code = KTT_B200_MASK_F32; break;
    }
    while (m.dim() < 4) m = m.unsqueeze(0);
    m = m.expand({b, h, sq, sk});
    a.mask = m.data_ptr();
    a.mask_dtype = code;
    for (int i = 0; i < 4; ++i) a.mask_strides[i] = m.stride(i);
    keep = m;
}

// The head-dim-64 forward's workspace: one zero-filled buffer per (device, stream); the kernel
// leaves it zero.
Tensor forward_workspace(const ktt_b200_attn_args& a, const Tensor& like, cudaStream_t stream) {
    const int64_t need = ktt_b200_sdpa_forward_workspace(&a);
    if (need <= 0) return Tensor();
    static std::mutex mu;
    static std::unordered_map<uint64_t, Tensor> cache;
    const uint64_t key = (static_cast<uint64_t>(like.get_device()) << 56) ^ reinterpret_cast<uint64_t>(stream);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end() || it->second.numel() < need) {
        Tensor buf = at::zeros({need}, like.options().dtype(at::kByte));
        it = cache.insert_or_assign(key, buf).first;
    }
    return it->second;
}

void fill_common(ktt_b200_attn_args& a, const Tensor& q, const Tensor& k, const Tensor& v, bool is_causal, c10::optional<double> scale) {
    std::memset(&a, 0, sizeof(a));
    a.batch = static_cast<int32_t>(q.size(0));
    a.heads = static_cast<int32_t>(q.size(1));
    a.kv_heads = static_cast<int32_t>(k.size(1));
    a.sq = static_cast<int32_t>(q.size(2));
    a.sk = static_cast<int32_t>(k.size(2));
    a.d = static_cast<int32_t>(q.size(3));
    a.dv = static_cast<int32_t>(v.size(3));
    a.causal = is_causal ? KTT_B200_CAUSAL_TOP_LEFT : KTT_B200_CAUSAL_NONE;
    a.scale = static_cast<float>(scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(q.size(3))));
    a.kernel = g_kernel < 0 ? KTT_B200_KERNEL_AUTO : g_kernel;
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.v = v.data_ptr();
    set3(a.q_strides, q);
    set3(a.k_strides, k);
    set3(a.v_strides, v);
}

// Forward into `out` (already allocated in the overload's layout); returns lse [B, H, rows].
Tensor run_forward(const Tensor& q_, const Tensor& k_, const Tensor& v_, const c10::optional<Tensor>& mask, bool is_causal,
                   c10::optional<double> scale, Tensor& out, bool need_lse, int64_t lse_rows) {
    const Tensor q = rows_contiguous(q_), k = rows_contiguous(k_), v = rows_contiguous(v_);
    c10::cuda::CUDAGuard guard(q.device());
    ktt_b200_attn_args a;
    fill_common(a, q, k, v, is_causal, scale);
    Tensor keep;
    mask_operand(a, mask, q.size(0), q.size(1), q.size(2), k.size(2), keep);
    a.out = out.data_ptr();
    set3(a.out_strides, out);
    Tensor lse;
    if (need_lse) {
        lse = at::empty({q.size(0), q.size(1), lse_rows}, q.options().dtype(at::kFloat));
        a.lse = lse.data_ptr<float>();
        a.lse_strides[0] = lse.stride(0);
        a.lse_strides[1] = lse.stride(1);
        a.lse_strides[2] = 1;
    }
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    Tensor ws = forward_workspace(a, q, stream);
    if (ws.defined()) {
        a.workspace = ws.data_ptr();
        a.workspace_bytes = ws.numel();
    }
    raise_status(ktt_b200_sdpa_forward(&a, stream), "sdpa_forward");
    return lse;
}

std::tuple<Tensor, Tensor, Tensor> run_backward(const Tensor& dout_, const Tensor& q_, const Tensor& k_, const Tensor& v_,
                                                const Tensor& out_, const Tensor& lse, const c10::optional<Tensor>& mask,
                                                bool is_causal, c10::optional<double> scale) {
    const Tensor q = rows_contiguous(q_), k = rows_contiguous(k_), v = rows_contiguous(v_);
    const Tensor dout = rows_contiguous(dout_), out = rows_contiguous(out_);
    TORCH_CHECK_VALUE(lse.scalar_type() == at::kFloat && lse.dim() == 3 && lse.stride(2) == 1,
                      "kohaku_tt_b200: lse must be fp32 [B, H, rows] with unit row stride");
    c10::cuda::CUDAGuard guard(q.device());
    ktt_b200_attn_args a;
    fill_common(a, q, k, v, is_causal, scale);
    Tensor keep;
    mask_operand(a, mask, q.size(0), q.size(1), q.size(2), k.size(2), keep);
    Tensor dq = at::empty(q.sizes(), q.options()), dk = at::empty(k.sizes(), k.options()), dv = at::empty(v.sizes(), v.options());
    a.out = out.data_ptr();
    a.lse = lse.data_ptr<float>();
    a.dout = dout.data_ptr();
    a.dq = dq.data_ptr();
    a.dk = dk.data_ptr();
    a.dv_out = dv.data_ptr();
    set3(a.out_strides, out);
    a.lse_strides[0] = lse.stride(0);
    a.lse_strides[1] = lse.stride(1);
    a.lse_strides[2] = 1;
    set3(a.dout_strides, dout);
    set3(a.dq_strides, dq);
    set3(a.dk_strides, dk);
    set3(a.dv_strides, dv);
    const int64_t nbytes = ktt_b200_sdpa_backward_workspace(&a);
    if (nbytes <= 0) raise_status(KTT_B200_ERR_UNSUPPORTED, "sdpa_backward");
    Tensor work = at::empty({nbytes}, q.options().dtype(at::kByte));
    a.workspace = work.data_ptr();
    a.workspace_bytes = nbytes;
    raise_status(ktt_b200_sdpa_backward(&a, at::cuda::getCurrentCUDAStream()), "sdpa_backward");
    return {dq, dk, dv};
}

// Output laid out the way torch's meta kernels of the flash, cuDNN and overrideable overloads
// promise (empty_like(query): the query's stride order).
Tensor out_like(const Tensor& q, int64_t dv) {
    if (dv == q.size(3)) return at::empty_like(q);
    int order[4] = {0, 1, 2, 3};
    std::sort(order, order + 4, [&](int x, int y) { return q.stride(x) != q.stride(y) ? q.stride(x) > q.stride(y) : x < y; });
    const int64_t shape[4] = {q.size(0), q.size(1), q.size(2), dv};
    Tensor out = at::empty({shape[order[0]], shape[order[1]], shape[order[2]], shape[order[3]]}, q.options());
    int64_t perm[4];
    for (int i = 0; i < 4; ++i) perm[order[i]] = i;
    return out.permute({perm[0], perm[1], perm[2], perm[3]});
}

struct Bf16 {
    Tensor q, k, v;
    bool cast;
};

// fp32 inputs without gradients are cast at entry and the output cast back
// (aten_attention.cpp:400-415).
Bf16 as_bf16(const Tensor& q, const Tensor& k, const Tensor& v) {
    if (q.scalar_type() == at::kFloat) return {q.to(at::kBFloat16), k.to(at::kBFloat16), v.to(at::kBFloat16), true};
    return {q, k, v, false};
}

Tensor empty0(const Tensor& like, at::ScalarType dtype) { return at::empty({0}, like.options().dtype(dtype)); }

c10::optional<Tensor> bias_or_none(const Tensor& bias) {
    if (!bias.defined() || bias.numel() == 0) return c10::nullopt;
    return bias;
}

// Gradient of an additive bias: dS summed over the dims the bias broadcasts, recomputed with
// separate matmul / softmax steps as the reference's masked backward does
// (aten_attention.cpp:781-811).
Tensor bias_gradient(const Tensor& grad_out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& bias,
                     c10::optional<double> scale) {
    const int64_t rep = q.size(1) / k.size(1);
    const Tensor kf = k.to(at::kFloat).repeat_interleave(rep, 1), vf = v.to(at::kFloat).repeat_interleave(rep, 1);
    const double sc = scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(q.size(3)));
    const Tensor s = at::matmul(q.to(at::kFloat), kf.transpose(-1, -2)) * sc + bias.to(at::kFloat).clamp_min(-5e5);
    const Tensor p = at::softmax(s, -1);
    const Tensor dp = at::matmul(grad_out.to(at::kFloat), vf.transpose(-1, -2));
    Tensor ds = p * (dp - (dp * p).sum(-1, true));
    Tensor b4 = bias;
    while (b4.dim() < 4) b4 = b4.unsqueeze(0);
    std::vector<int64_t> dims;
    for (int64_t i = 0; i < 4; ++i) {
        if (b4.size(i) == 1 && ds.size(i) != 1) dims.push_back(i);
    }
    if (!dims.empty()) ds = ds.sum(dims, true);
    return ds.reshape(bias.sizes()).to(bias.scalar_type());
}

// ---- the overloads ---------------------------------------------------------------------------

std::tuple<Tensor, Tensor, Tensor, Tensor, c10::SymInt, c10::SymInt, Tensor, Tensor, Tensor> flash_forward(
    const Tensor& q, const Tensor& k, const Tensor& v, double dropout_p, bool is_causal, bool /*return_debug_mask*/,
    c10::optional<double> scale) {
    checked(q, k, v, c10::nullopt, dropout_p, is_causal);
    const Bf16 x = as_bf16(q, k, v);
    Tensor out = out_like(x.q, x.v.size(3));
    Tensor lse = run_forward(x.q, x.k, x.v, c10::nullopt, is_causal, scale, out, true, q.size(2));
    if (x.cast) out = out.to(at::kFloat);
    // Dropout is refused, so nobody reads the generator state: left unwritten.
    return {out, lse, empty0(q, at::kLong), empty0(q, at::kLong), c10::SymInt(q.size(2)), c10::SymInt(k.size(2)),
            at::empty({2}, q.options().dtype(at::kUInt64)), at::empty({}, q.options().dtype(at::kUInt64)),
            empty0(q, q.scalar_type())};
}

std::tuple<Tensor, Tensor, Tensor> flash_backward(
    const Tensor& grad_out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse,
    const Tensor&, const Tensor&, c10::SymInt, c10::SymInt, double dropout_p, bool is_causal, const Tensor&, const Tensor&,
    c10::optional<double> scale) {
    checked(q, k, v, c10::nullopt, dropout_p, is_causal);
    return run_backward(grad_out, q, k, v, out, lse, c10::nullopt, is_causal, scale);
}

std::tuple<Tensor, Tensor, Tensor, Tensor> efficient_forward(
    const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& bias, bool compute_lse, double dropout_p,
    bool is_causal, c10::optional<double> scale) {
    checked(q, k, v, bias, dropout_p, is_causal);
    const Bf16 x = as_bf16(q, k, v);
    // The efficient overload's meta promises [B, Sq, H, Dv] storage seen as [B, H, Sq, Dv].
    Tensor out = at::empty({q.size(0), q.size(2), q.size(1), v.size(3)}, x.q.options()).transpose(1, 2);
    const int64_t rows = (q.size(2) + 31) / 32 * 32;
    Tensor lse = run_forward(x.q, x.k, x.v, bias, is_causal, scale, out, compute_lse, rows);
    if (!lse.defined()) lse = at::empty({q.size(0), q.size(1), 0}, q.options().dtype(at::kFloat));
    if (x.cast) out = out.to(at::kFloat);
    return {out, lse, at::empty({}, q.options().dtype(at::kLong)), at::empty({}, q.options().dtype(at::kLong))};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> efficient_backward(
    const Tensor& grad_out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& bias_, const Tensor& out,
    const Tensor& lse, const Tensor&, const Tensor&, double dropout_p, std::array<bool, 4> grad_input_mask, bool is_causal,
    c10::optional<double> scale) {
    const c10::optional<Tensor> bias = bias_or_none(bias_);
    checked(q, k, v, bias, dropout_p, is_causal);
    auto [dq, dk, dv] = run_backward(grad_out, q, k, v, out, lse, bias, is_causal, scale);
    Tensor dbias;
    if (bias.has_value() && grad_input_mask[3]) dbias = bias_gradient(grad_out, q, k, v, *bias, scale);
    return {dq, dk, dv, dbias};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, c10::SymInt, c10::SymInt, Tensor, Tensor, Tensor> cudnn_forward(
    const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& bias, bool /*compute_lse*/, double dropout_p,
    bool is_causal, bool /*return_debug_mask*/, c10::optional<double> scale) {
    checked(q, k, v, bias, dropout_p, is_causal);
    const Bf16 x = as_bf16(q, k, v);
    Tensor out = out_like(x.q, x.v.size(3));
    Tensor lse = run_forward(x.q, x.k, x.v, bias, is_causal, scale, out, true, q.size(2));
    if (x.cast) out = out.to(at::kFloat);
    return {out, lse.unsqueeze(-1), empty0(q, at::kLong), empty0(q, at::kLong), c10::SymInt(q.size(2)), c10::SymInt(k.size(2)),
            at::empty({}, q.options().dtype(at::kLong)), at::empty({}, q.options().dtype(at::kLong)), empty0(q, q.scalar_type())};
}

std::tuple<Tensor, Tensor, Tensor> cudnn_backward(
    const Tensor& grad_out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse_,
    const Tensor&, const Tensor&, const Tensor& bias_, const Tensor&, const Tensor&, c10::SymInt, c10::SymInt, double dropout_p,
    bool is_causal, c10::optional<double> scale) {
    const c10::optional<Tensor> bias = bias_or_none(bias_);
    checked(q, k, v, bias, dropout_p, is_causal);
    const Tensor lse = (lse_.dim() == 4 ? lse_.squeeze(-1) : lse_).contiguous();
    return run_backward(grad_out, q, k, v, out, lse, bias, is_causal, scale);
}

std::tuple<Tensor, Tensor, Tensor, Tensor, c10::SymInt, c10::SymInt, Tensor, Tensor, Tensor> overrideable_forward(
    const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& bias, double dropout_p, bool is_causal,
    bool /*return_debug_mask*/, c10::optional<double> scale) {
    checked(q, k, v, bias, dropout_p, is_causal);
    const Bf16 x = as_bf16(q, k, v);
    Tensor out = out_like(x.q, x.v.size(3));
    Tensor lse = run_forward(x.q, x.k, x.v, bias, is_causal, scale, out, true, q.size(2));
    if (x.cast) out = out.to(at::kFloat);
    return {out, lse, empty0(q, at::kLong), empty0(q, at::kLong), c10::SymInt(q.size(2)), c10::SymInt(k.size(2)),
            at::empty({}, q.options().dtype(at::kLong)), at::empty({}, q.options().dtype(at::kLong)), empty0(q, q.scalar_type())};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> overrideable_backward(
    const Tensor& grad_out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& bias_,
    std::array<bool, 4> grad_input_mask, const Tensor& out, const Tensor& lse, const Tensor&, const Tensor&, c10::SymInt,
    c10::SymInt, double dropout_p, bool is_causal, const Tensor&, const Tensor&, c10::optional<double> scale) {
    const c10::optional<Tensor> bias = bias_or_none(bias_);
    checked(q, k, v, bias, dropout_p, is_causal);
    auto [dq, dk, dv] = run_backward(grad_out, q, k, v, out, lse, bias, is_causal, scale);
    Tensor dbias = empty0(q, q.scalar_type());
    if (bias.has_value() && grad_input_mask[3]) dbias = bias_gradient(grad_out, q, k, v, *bias, scale);
    return {dq, dk, dv, dbias};
}

// SDPBackend: MATH 0, OVERRIDEABLE 4. MATH when torch's own switch has every fused backend
// whose overload lands here turned off (the reference asks the one switch its overload sits
// behind, aten_attention.cpp:204-207), or when the shapes are refused.
int64_t fused_sdp_choice(const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& mask, double dropout_p,
                         bool is_causal, c10::optional<double> /*scale*/, bool /*enable_gqa*/) {
    auto& ctx = at::globalContext();
    if (!(ctx.userEnabledFlashSDP() || ctx.userEnabledMemEfficientSDP() || ctx.userEnabledCuDNNSDP() || ctx.userEnabledOverrideableSDP())) {
        return 0;
    }
    return fused_refusal(q, k, v, mask, dropout_p, is_causal) ? 0 : 4;
}

std::unique_ptr<torch::Library> g_library;
std::mutex g_install_mutex;

}  // namespace

extern "C" {

__attribute__((visibility("default"))) int ktt_b200_aten_install(void) {
    std::lock_guard<std::mutex> lock(g_install_mutex);
    if (g_library) return 0;
    try {
        auto lib = std::make_unique<torch::Library>(torch::Library::IMPL, "aten", c10::make_optional(c10::DispatchKey::CUDA), __FILE__, __LINE__);
        lib->impl("_scaled_dot_product_flash_attention", TORCH_FN(flash_forward));
        lib->impl("_scaled_dot_product_flash_attention_backward", TORCH_FN(flash_backward));
        lib->impl("_scaled_dot_product_efficient_attention", TORCH_FN(efficient_forward));
        lib->impl("_scaled_dot_product_efficient_attention_backward", TORCH_FN(efficient_backward));
        lib->impl("_scaled_dot_product_cudnn_attention", TORCH_FN(cudnn_forward));
        lib->impl("_scaled_dot_product_cudnn_attention_backward", TORCH_FN(cudnn_backward));
        lib->impl("_scaled_dot_product_fused_attention_overrideable", TORCH_FN(overrideable_forward));
        lib->impl("_scaled_dot_product_fused_attention_overrideable_backward", TORCH_FN(overrideable_backward));
        lib->impl("_fused_sdp_choice", TORCH_FN(fused_sdp_choice));
        g_library = std::move(lib);
    } catch (const std::exception&) {
        return -1;
    }
    return 0;
}

__attribute__((visibility("default"))) int ktt_b200_aten_uninstall(void) {
    std::lock_guard<std::mutex> lock(g_install_mutex);
    g_library.reset();
    return 0;
}

// The calling thread's kernel scope: `kernel` is a KTT_B200_KERNEL_* code or -1 (the scope
// allows no kernel); `names` the scope's kernel list for error messages ("" outside a scope).
__attribute__((visibility("default"))) void ktt_b200_aten_set_scope(int kernel, const char* names) {
    g_kernel = kernel;
    g_scope_names = names ? names : "";
}

}  // extern "C"
