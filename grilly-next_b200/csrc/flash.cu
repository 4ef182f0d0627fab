// grl_flash_fwd: argument checks and kernel choice for the prefill path.
#include "common.cuh"

namespace grl {
int flash_fwd_simt(grl_device* dev, const grl_flash_params* p, float scale, const float2* rope);
int flash_fwd_sm100(grl_device* dev, const grl_flash_params* p, float scale, const float2* rope, int32_t* status);
}  // namespace grl

using namespace grl;

extern "C" int grl_flash_fwd(grl_device* dev, const grl_flash_params* p) {
    GRL_REQUIRE(dev && p, "NULL argument");
    GRL_REQUIRE(p->q && p->k && p->v && p->o, "NULL tensor pointer");
    GRL_REQUIRE(p->batch > 0 && p->heads > 0 && p->seq_len > 0 && p->head_dim > 0, "bad shape (%d,%d,%d,%d)",
                p->batch, p->heads, p->seq_len, p->head_dim);
    GRL_REQUIRE(p->in_dtype == GRL_F32 || p->in_dtype == GRL_BF16, "unknown in_dtype");
    GRL_REQUIRE(p->out_dtype == GRL_F32 || p->out_dtype == GRL_BF16, "unknown out_dtype");
    GRL_REQUIRE(p->rope_mode >= GRL_ROPE_NONE && p->rope_mode <= GRL_ROPE_HALF, "unknown rope mode");
    GRL_REQUIRE(!p->mask || (p->mask_kind >= GRL_MASK_KEY && p->mask_kind <= GRL_MASK_BHSS), "unknown mask kind");
    GRL_REQUIRE(p->head_dim % 2 == 0, "head_dim must be even");
    DeviceGuard g(dev->ordinal);
    const float scale = p->scale == 0.f ? 1.f / sqrtf((float)p->head_dim) : p->scale;

    const float2* rope = nullptr;
    if (p->rope_mode != GRL_ROPE_NONE) {
        GRL_REQUIRE(p->rope_theta > 0.f, "rope_theta must be positive");
        int rc = get_rope_table(dev, p->seq_len, p->head_dim, p->rope_theta,
                                p->rope_scaling == 0.f ? 1.f : p->rope_scaling, &rope);
        if (rc) return rc;
    }

    int kernel = p->kernel;
    if (kernel == GRL_KERNEL_AUTO)
        kernel = (p->in_dtype == GRL_BF16 && (p->head_dim == 128 || p->head_dim == 64) && !p->mask && scale > 0.f) ? GRL_KERNEL_TCGEN05
                                                                                            : GRL_KERNEL_SIMT_F32;
    if (kernel == GRL_KERNEL_SIMT_F32) return flash_fwd_simt(dev, p, scale, rope);
    if (kernel == GRL_KERNEL_TCGEN05) {
        int32_t* status = p->status ? p->status : dev->d_status;
        if (!p->status) dev->status_dirty = true;
        return flash_fwd_sm100(dev, p, scale, rope, status);
    }
    return set_error(GRL_ERR_INVALID, "unknown kernel selector %d", kernel);
}
