// PyTorch C++ extension over the C ABI of include/vqattn.h: registers the library's entry points as
// dispatcher operators (torch.ops.vqattn.*), so that a PyTorch program can call them like any other
// operator - under a device guard, on PyTorch's current stream, with TORCH_CHECK errors - without going
// through Python's ctypes.  Nothing here computes: every operator describes its tensors as VqTensorDesc,
// calls the C function the header declares and turns a negative status into an exception.  All operators
// write into tensors the caller passes (out-variants): the library allocates nothing, and neither does
// this file.
//
// Reference interfaces behind the operators: ops/mini_vq.py:4-18 (assign_codes), ops/attn_vq.py:352-384,
// 411-417 (build_aggregates), ops/triton_fused_vq_attn.py:190-251 (prefill), README.md:8 and
// ops/attn_vq.py:128-165 (decode, cache_advance).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <optional>

#include "vqattn.h"

namespace {

int32_t dtype_of(const at::Tensor &t)
{
    switch (t.scalar_type()) {
        case at::kFloat: return VQ_F32;
        case at::kBFloat16: return VQ_BF16;
        case at::kHalf: return VQ_F16;
        case at::kByte: return VQ_U8;
        case at::kUInt16: return VQ_U16;
        case at::kInt: return VQ_I32;
        case at::kLong: return VQ_I64;
        default: TORCH_CHECK(false, "vqattn: unsupported dtype ", t.scalar_type());
    }
    return -1;
}

VqTensorDesc desc(const at::Tensor &t)
{
    TORCH_CHECK(t.is_cuda(), "vqattn: CUDA tensors only (there is no CPU path)");
    TORCH_CHECK(t.dim() <= VQATTN_MAX_DIMS, "vqattn: at most ", VQATTN_MAX_DIMS, " dimensions");
    VqTensorDesc d{};
    d.ptr = t.data_ptr();
    d.dtype = dtype_of(t);
    d.ndim = static_cast<int32_t>(t.dim());
    for (int64_t i = 0; i < t.dim(); ++i) {
        d.shape[i] = t.size(i);
        d.stride[i] = t.stride(i);
    }
    d.device = static_cast<int32_t>(t.get_device());
    return d;
}

VqTensorDesc desc(const std::optional<at::Tensor> &t)
{
    if (t.has_value() && t->defined()) return desc(*t);
    VqTensorDesc d{};
    d.device = -1;
    return d;
}

void check(int status, const char *where)
{
    TORCH_CHECK(status == VQ_OK, where, ": ", vqattn_status_string(status), " (status ", status, ")");
}

void *stream_of(const at::Tensor &t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

int32_t *word_of(const std::optional<at::Tensor> &w)
{
    if (!w.has_value() || !w->defined()) return nullptr;
    TORCH_CHECK(w->is_cuda() && w->scalar_type() == at::kInt && w->numel() >= 1, "vqattn: status word must be a CUDA int32 tensor");
    return w->data_ptr<int32_t>();
}

struct Workspace {
    void *ptr = nullptr;
    size_t bytes = 0;
    explicit Workspace(const std::optional<at::Tensor> &w)
    {
        if (w.has_value() && w->defined()) {
            TORCH_CHECK(w->is_cuda() && w->is_contiguous(), "vqattn: workspace must be a contiguous CUDA tensor");
            ptr = w->data_ptr();
            bytes = static_cast<size_t>(w->numel()) * w->element_size();
        }
    }
};

// codes[B,Hkv,L,M] <- assignment of k[B,Hkv,L,D] against codebooks[Hkv,M,K,D]; with a workspace of
// assign_workspace_bytes(...) the scores run on the tensor cores (same codes)
void assign_codes(const at::Tensor &k, const at::Tensor &codebooks, const std::optional<at::Tensor> &bias, at::Tensor codes,
                  const std::optional<at::Tensor> &workspace, const std::optional<at::Tensor> &status_word)
{
    const c10::cuda::CUDAGuard guard(k.device());
    VqTensorDesc dk = desc(k), dc = desc(codebooks), db = desc(bias), dout = desc(codes);
    const Workspace ws(workspace);
    const VqTensorDesc *pb = (bias.has_value() && bias->defined()) ? &db : nullptr;
    if (ws.ptr != nullptr)
        check(vqattn_assign_codes_ws(&dk, &dc, pb, &dout, ws.ptr, ws.bytes, word_of(status_word), stream_of(k)), "vqattn::assign_codes");
    else
        check(vqattn_assign_codes(&dk, &dc, pb, &dout, stream_of(k)), "vqattn::assign_codes");
}

int64_t assign_workspace_bytes(int64_t B, int64_t Hkv, int64_t L, int64_t M, int64_t K, int64_t D)
{
    return static_cast<int64_t>(vqattn_assign_workspace_bytes(B, Hkv, L, M, K, D));
}

// cnt[B,Hkv,NB,MK], vsum[B,Hkv,NB,MK,D] <- per-block aggregates; state_cnt / state_vsum (both or neither): the fp32
// aggregates of the first state_blocks * 128 keys from the same pass
void build_aggregates(const at::Tensor &codes, const at::Tensor &v, int64_t K, at::Tensor cnt, at::Tensor vsum,
                      const std::optional<at::Tensor> &state_cnt, const std::optional<at::Tensor> &state_vsum, int64_t state_blocks,
                      const std::optional<at::Tensor> &workspace, const std::optional<at::Tensor> &status_word)
{
    const c10::cuda::CUDAGuard guard(v.device());
    VqTensorDesc dc = desc(codes), dv = desc(v), dcnt = desc(cnt), dvs = desc(vsum);
    const Workspace ws(workspace);
    const bool with_state = state_cnt.has_value() && state_cnt->defined();
    TORCH_CHECK(with_state == (state_vsum.has_value() && state_vsum->defined()), "vqattn::build_aggregates: pass both state tensors or neither");
    if (with_state) {
        VqTensorDesc dsc = desc(state_cnt), dsv = desc(state_vsum);
        check(vqattn_build_aggregates_state(&dc, &dv, static_cast<int32_t>(K), &dcnt, &dvs, &dsc, &dsv, state_blocks, ws.ptr, ws.bytes,
                                            word_of(status_word), stream_of(v)),
              "vqattn::build_aggregates");
    } else {
        check(vqattn_build_aggregates_ws(&dc, &dv, static_cast<int32_t>(K), &dcnt, &dvs, ws.ptr, ws.bytes, word_of(status_word), stream_of(v)),
              "vqattn::build_aggregates");
    }
}

int64_t aggregates_workspace_bytes(int64_t B, int64_t Hkv, int64_t NB, int64_t M, int64_t K)
{
    return static_cast<int64_t>(vqattn_aggregates_workspace_bytes(B, Hkv, NB, M, K));
}

// out[B,Hq,L,D] <- fused prefill attention (window keys exactly, older keys through the aggregates)
void prefill(const at::Tensor &q1, const at::Tensor &q2, const at::Tensor &k1, const at::Tensor &k3, const at::Tensor &v,
             const std::optional<at::Tensor> &codebook, const std::optional<at::Tensor> &cnt, const std::optional<at::Tensor> &vsum,
             int64_t window, double scale, int64_t impl, at::Tensor out, const std::optional<at::Tensor> &lse2,
             const std::optional<at::Tensor> &status_word)
{
    const c10::cuda::CUDAGuard guard(q1.device());
    VqPrefillArgs a{};
    a.q1 = desc(q1); a.q2 = desc(q2); a.k1 = desc(k1); a.k3 = desc(k3); a.v = desc(v);
    a.codebook = desc(codebook); a.cnt = desc(cnt); a.vsum = desc(vsum);
    a.out = desc(out);
    a.lse2 = desc(lse2);
    a.window = window;
    a.scale = static_cast<float>(scale);
    a.impl = static_cast<int32_t>(impl);
    a.status_word = word_of(status_word);
    check(vqattn_prefill(&a, stream_of(q1)), "vqattn::prefill");
}

// out[B,Hq,D] <- one decode step over the window caches and the aggregates
void decode(const at::Tensor &q1, const at::Tensor &q2, const at::Tensor &k1_win, const at::Tensor &k3_win, const at::Tensor &v_win,
            const std::optional<at::Tensor> &codebook, const std::optional<at::Tensor> &cnt, const std::optional<at::Tensor> &vsum,
            int64_t n_valid, int64_t n_bd, double scale, at::Tensor workspace, at::Tensor out, const std::optional<at::Tensor> &status_word)
{
    const c10::cuda::CUDAGuard guard(q1.device());
    VqDecodeArgs a{};
    a.q1 = desc(q1); a.q2 = desc(q2); a.k1_win = desc(k1_win); a.k3_win = desc(k3_win); a.v_win = desc(v_win);
    a.codebook = desc(codebook); a.cnt = desc(cnt); a.vsum = desc(vsum);
    a.out = desc(out);
    a.n_valid = n_valid;
    a.n_bd = n_bd;
    a.use_far = (codebook.has_value() && codebook->defined()) ? 1 : 0;
    a.scale = static_cast<float>(scale);
    const std::optional<at::Tensor> ws_t{workspace};
    const Workspace ws(ws_t);
    a.workspace = ws.ptr;
    a.workspace_bytes = ws.bytes;
    a.status_word = word_of(status_word);
    check(vqattn_decode(&a, stream_of(q1)), "vqattn::decode");
}

int64_t decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t D)
{
    return static_cast<int64_t>(vqattn_decode_workspace_bytes(B, Hq, Hkv, D));
}

// cnt[B,Hkv,MK], vsum_f32[B,Hkv,MK,D] (+ 16-bit copy) += the keys codes[B,Hkv,n,M] / v_new[B,Hkv,n,D] that left the window
void cache_advance(const at::Tensor &codes, const at::Tensor &v_new, int64_t K, at::Tensor cnt, at::Tensor vsum_f32,
                   const std::optional<at::Tensor> &vsum_act, const std::optional<at::Tensor> &status_word)
{
    const c10::cuda::CUDAGuard guard(v_new.device());
    VqTensorDesc dc = desc(codes), dv = desc(v_new), dcnt = desc(cnt), dvs = desc(vsum_f32), dva = desc(vsum_act);
    VqTensorDesc *pva = (vsum_act.has_value() && vsum_act->defined()) ? &dva : nullptr;
    check(vqattn_cache_advance(&dc, &dv, static_cast<int32_t>(K), &dcnt, &dvs, pva, word_of(status_word), stream_of(v_new)),
          "vqattn::cache_advance");
}

int64_t abi_version() { return vqattn_version(); }

}  // namespace

TORCH_LIBRARY(vqattn, m)
{
    m.def("abi_version() -> int", &abi_version);
    m.def("assign_workspace_bytes(int B, int Hkv, int L, int M, int K, int D) -> int", &assign_workspace_bytes);
    m.def("aggregates_workspace_bytes(int B, int Hkv, int NB, int M, int K) -> int", &aggregates_workspace_bytes);
    m.def("decode_workspace_bytes(int B, int Hq, int Hkv, int D) -> int", &decode_workspace_bytes);
    m.def("assign_codes(Tensor k, Tensor codebooks, Tensor? bias, Tensor(a!) codes, Tensor(b!)? workspace, Tensor(c!)? status_word) -> ()");
    m.def("build_aggregates(Tensor codes, Tensor v, int K, Tensor(a!) cnt, Tensor(b!) vsum, Tensor(c!)? state_cnt, Tensor(d!)? state_vsum, "
          "int state_blocks, Tensor(e!)? workspace, Tensor(f!)? status_word) -> ()");
    m.def("prefill(Tensor q1, Tensor q2, Tensor k1, Tensor k3, Tensor v, Tensor? codebook, Tensor? cnt, Tensor? vsum, int window, "
          "float scale, int impl, Tensor(a!) out, Tensor(b!)? lse2, Tensor(c!)? status_word) -> ()");
    m.def("decode(Tensor q1, Tensor q2, Tensor k1_win, Tensor k3_win, Tensor v_win, Tensor? codebook, Tensor? cnt, Tensor? vsum, "
          "int n_valid, int n_bd, float scale, Tensor(a!) workspace, Tensor(b!) out, Tensor(c!)? status_word) -> ()");
    m.def("cache_advance(Tensor codes, Tensor v_new, int K, Tensor(a!) cnt, Tensor(b!) vsum_f32, Tensor(c!)? vsum_act, "
          "Tensor(d!)? status_word) -> ()");
}

TORCH_LIBRARY_IMPL(vqattn, CUDA, m)
{
    m.impl("assign_codes", &assign_codes);
    m.impl("build_aggregates", &build_aggregates);
    m.impl("prefill", &prefill);
    m.impl("decode", &decode);
    m.impl("cache_advance", &cache_advance);
}
