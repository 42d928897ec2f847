// C-ABI entry points that only validate and dispatch: version, status strings, the wait bound, prefill.
#include <atomic>

#include "tc_ptx.cuh"
#include "vq_common.cuh"

namespace vq {
int launch_prefill_simt(const VqPrefillArgs *a, cudaStream_t stream);
int launch_prefill_tensor4(const VqPrefillArgs *a, cudaStream_t stream);
}  // namespace vq

namespace vq {

static std::atomic<long long> g_wait_limit{ptx::kDefaultWaitCycles};
long long wait_limit_cycles() { return g_wait_limit.load(std::memory_order_relaxed); }

// One CTA waits on a barrier that nothing ever arrives at: the wait must give up after `limit` cycles.
__global__ void wait_selftest_kernel(long long limit, int32_t *status)
{
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_mbar_init();
        if (!ptx::mbar_wait(&bar, 0, limit) && status) atomicExch(status, VQ_WORD_TIMEOUT);
    }
}

}  // namespace vq

extern "C" int vqattn_version(void) { return VQATTN_VERSION; }

extern "C" int vqattn_status_from_word(int32_t word)
{
    switch (word) {
    case 0: return VQ_OK;
    case VQ_WORD_TIMEOUT: return VQ_ETIMEOUT;
    case VQ_WORD_BAD_POSITION:
    case VQ_WORD_BAD_CODE: return VQ_EINVAL_ARG;
    default: return VQ_ELAUNCH;
    }
}

extern "C" int64_t vqattn_set_wait_limit_cycles(int64_t cycles)
{
    return vq::g_wait_limit.exchange(cycles > 0 ? cycles : vq::ptx::kDefaultWaitCycles);
}

extern "C" int vqattn_wait_selftest(int32_t *status_word, void *stream)
{
    if (status_word == nullptr) return VQ_EINVAL_ARG;
    vq::wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(vq::wait_limit_cycles(), status_word);
    return vq::launch_status();
}

extern "C" const char *vqattn_status_string(int status)
{
    switch (status) {
    case VQ_OK: return "ok";
    case VQ_EINVAL_SHAPE: return "invalid shape";
    case VQ_EINVAL_DTYPE: return "invalid dtype";
    case VQ_EINVAL_STRIDE: return "invalid stride or alignment";
    case VQ_EDEVICE: return "tensor not on the current CUDA device";
    case VQ_ELAUNCH: return "CUDA launch failed";
    case VQ_ETIMEOUT: return "device-side wait timed out";
    case VQ_EINVAL_ARG: return "invalid argument";
    case VQ_EUNSUPPORTED: return "unsupported configuration";
    case VQ_EWORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
    }
}

extern "C" int vqattn_prefill(const VqPrefillArgs *a, void *stream)
{
    using namespace vq;
    if (a == nullptr) return VQ_EINVAL_ARG;
    int st;
    const VqTensorDesc *qs[] = {&a->q1, &a->q2, &a->out};
    const VqTensorDesc *ks[] = {&a->k1, &a->k3, &a->v};
    for (auto t : qs)
        if ((st = check_basic(t, 4)) != VQ_OK) return st;
    for (auto t : ks)
        if ((st = check_basic(t, 4)) != VQ_OK) return st;
    const int64_t B = a->q1.shape[0], Hq = a->q1.shape[1], L = a->q1.shape[2], D = a->q1.shape[3];
    const int64_t Hkv = a->k1.shape[1];
    const int dt = a->q1.dtype;
    if (!is_act_dtype(dt)) return VQ_EINVAL_DTYPE;
    if (Hkv <= 0 || Hq % Hkv != 0) return VQ_EINVAL_SHAPE;
    for (auto t : qs) {
        if (t->dtype != dt) return VQ_EINVAL_DTYPE;
        if (t->shape[0] != B || t->shape[1] != Hq || t->shape[2] != L || t->shape[3] != D) return VQ_EINVAL_SHAPE;
    }
    for (auto t : ks) {
        if (t->dtype != dt) return VQ_EINVAL_DTYPE;
        if (t->shape[0] != B || t->shape[1] != Hkv || t->shape[2] != L || t->shape[3] != D) return VQ_EINVAL_SHAPE;
    }
    if (a->window <= 0 || a->window % kBlock != 0) return VQ_EINVAL_ARG;
    if (D != 64 && D != 128) return VQ_EUNSUPPORTED;
    // far blocks needed: query tile t (rows 128t..) with 128t - window > 0 reads block t - window/128 - 1
    const int64_t tiles = (L + kBlock - 1) / kBlock;
    const int64_t need_nb = tiles - a->window / kBlock - 1;
    const bool far = need_nb > 0 && a->codebook.ptr != nullptr;  // NULL codebook: local attention only
    if (far) {
        if ((st = check_basic(&a->codebook, 3)) != VQ_OK) return st;
        if ((st = check_basic(&a->cnt, 4)) != VQ_OK) return st;
        if ((st = check_basic(&a->vsum, 5)) != VQ_OK) return st;
        const int64_t MK = a->codebook.shape[1], NB = a->cnt.shape[2];
        if (a->codebook.dtype != dt || a->vsum.dtype != dt || a->cnt.dtype != VQ_F32) return VQ_EINVAL_DTYPE;
        if (a->codebook.shape[0] != Hkv || a->codebook.shape[2] != D) return VQ_EINVAL_SHAPE;
        if (MK % kBlock != 0) return VQ_EUNSUPPORTED;
        if (a->cnt.shape[0] != B || a->cnt.shape[1] != Hkv || a->cnt.shape[3] != MK) return VQ_EINVAL_SHAPE;
        if (a->vsum.shape[0] != B || a->vsum.shape[1] != Hkv || a->vsum.shape[2] != NB || a->vsum.shape[3] != MK ||
            a->vsum.shape[4] != D)
            return VQ_EINVAL_SHAPE;
        if (NB < need_nb) return VQ_EINVAL_SHAPE;
        if (!is_dense(a->codebook) || !is_dense(a->cnt) || !is_dense(a->vsum)) return VQ_EINVAL_STRIDE;
        if (reinterpret_cast<uintptr_t>(a->codebook.ptr) % 16 || reinterpret_cast<uintptr_t>(a->vsum.ptr) % 16 ||
            reinterpret_cast<uintptr_t>(a->cnt.ptr) % 16)
            return VQ_EINVAL_STRIDE;
    }
    if (a->lse2.ptr != nullptr) {
        if (a->lse2.ndim != 3 || a->lse2.dtype != VQ_F32 || !is_dense(a->lse2)) return VQ_EINVAL_SHAPE;
        if (a->lse2.shape[0] != B || a->lse2.shape[1] != Hq || a->lse2.shape[2] != L) return VQ_EINVAL_SHAPE;
    }
    const VqTensorDesc *all[] = {&a->q1, &a->q2, &a->out, &a->k1, &a->k3, &a->v, far ? &a->codebook : nullptr,
                                 far ? &a->cnt : nullptr, far ? &a->vsum : nullptr, a->lse2.ptr ? &a->lse2 : nullptr};
    if ((st = check_device(all, 10)) != VQ_OK) return st;
    const int64_t row_align = dt == VQ_F32 ? 4 : 8;
    const VqTensorDesc *rows[] = {&a->q1, &a->q2, &a->out, &a->k1, &a->k3, &a->v};
    for (auto t : rows) {
        if (t->stride[0] % row_align || t->stride[1] % row_align || t->stride[2] % row_align) return VQ_EINVAL_STRIDE;
        if (reinterpret_cast<uintptr_t>(t->ptr) % 16) return VQ_EINVAL_STRIDE;
    }
    if (B * Hq > 65535) return VQ_EUNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int impl = a->impl;
    if (impl == VQ_IMPL_AUTO) impl = is_16bit(dt) ? VQ_IMPL_TENSOR : VQ_IMPL_SIMT;
    if (impl == VQ_IMPL_SIMT) return launch_prefill_simt(a, s);
    if (impl == VQ_IMPL_TENSOR) {
        if (!is_16bit(dt)) return VQ_EINVAL_DTYPE;
        return launch_prefill_tensor4(a, s);
    }
    return VQ_EINVAL_ARG;
}
