// Cross-GPU log-sum-exp merge over NVLink peer memory: the exchange step of the KV-sharded
// long-context decode, fused with the merge.
//
// Every rank holds one un-normalised partial [O (rows*D) | m (rows) | l (rows)] of its KV shard.
// Instead of an all-gather followed by a merge, ONE kernel per rank (a) stores the local partial
// straight into every peer's inbox (plain st.global through NVLink, then a system-scope fence and
// a flag with the step's sequence number), (b) waits -- bounded -- for the peers' flags in its own
// inbox, and (c) merges.  The reference has no multi-GPU code; the merge arithmetic is that of
// lse_merge_kernel.  Inboxes are double-buffered by step parity: a rank can be at most one step
// ahead of a peer (it needs that peer's partial to finish a step), so the slot it overwrites was
// consumed two steps ago.  No TMA, no multicast, no multimem: ordinary peer loads/stores only.
#include <string.h>

#include "common.cuh"

namespace grl {

struct ExchangeArgs {
    const float* local_part;       // this rank's partial (n floats)
    PeerExchange x;                // seq already bumped for this step
    float* out;                    // (rows, D)
    int32_t* status;
    int rows, D;
};

int fill_peer_exchange(grl_device* dev, const grl_exchange_params* p, PeerExchange* x) {
    GRL_REQUIRE(p->world >= 1 && p->world <= kMaxPeers && p->rank >= 0 && p->rank < p->world, "bad rank / world");
    GRL_REQUIRE(p->inbox && p->flags && p->seq, "NULL buffer");
    GRL_REQUIRE(p->peer_inbox && p->peer_flags, "NULL peer tables");
    GRL_REQUIRE((uintptr_t)p->inbox % 16 == 0, "inbox must be 16-byte aligned");
    x->inbox = p->inbox; x->flags = p->flags; x->seq = p->seq;
    x->rank = p->rank; x->world = p->world; x->flag_slots = p->flag_slots > 0 ? p->flag_slots : 1;
    x->wait_cycles = p->wait_cycles > 0 ? (long long)p->wait_cycles : dev->peer_wait_limit_cycles;
    for (int r = 0; r < p->world; ++r) {
        GRL_REQUIRE(r == p->rank || (p->peer_inbox[r] && p->peer_flags[r]), "peer %d has no inbox", r);
        x->peer_inbox[r] = p->peer_inbox[r];
        x->peer_flags[r] = p->peer_flags[r];
    }
    return GRL_OK;
}

__global__ void bump_seq_kernel(unsigned int* seq) { *seq += 1; }

// grid = rows CTAs of 128 threads.  CTA p < world, p != rank, first pushes to peer p.
__global__ void __launch_bounds__(128) exchange_merge_kernel(ExchangeArgs a) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const PeerExchange& x = a.x;
    const unsigned int e = *x.seq;
    const int par = e & 1;
    const size_t n = (size_t)a.rows * (a.D + 2);
    if (row < x.world && row != x.rank) {
        float* dst = x.peer_inbox[row] + ((size_t)par * x.world + x.rank) * n;
        const float4* src4 = reinterpret_cast<const float4*>(a.local_part);
        float4* dst4 = reinterpret_cast<float4*>(dst);
        for (size_t i = tid; i < n / 4; i += 128) dst4[i] = src4[i];
        for (size_t i = (n / 4) * 4 + tid; i < n; i += 128) dst[i] = a.local_part[i];
        __threadfence_system();
        __syncthreads();
        if (tid == 0) {
            volatile unsigned int* f = x.peer_flags[row] + (size_t)(par * x.world + x.rank) * x.flag_slots;
            *f = e;
            __threadfence_system();
        }
    }
    // wait for every peer's partial of this step: lane r of the first warp watches peer r, so that the flags
    // are polled side by side and the wait costs one round trip past the slowest peer
    __shared__ int s_ok;
    if (tid < 32) {
        bool ok = true;
        if (tid < x.world && tid != x.rank) {
            const long long t0 = clock64();
            volatile unsigned int* f = x.flags + (size_t)(par * x.world + tid) * x.flag_slots;
            while (*f != e) {
                if (clock64() - t0 > x.wait_cycles) {
                    ok = false;
                    if (a.status && atomicCAS(a.status, 0, GRL_ERR_TIMEOUT) == 0) {
                        a.status[1] = (3 << 28) | tid;
                        a.status[2] = (int)e;
                        a.status[3] = x.rank;
                    }
                    break;
                }
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        __threadfence_system();
        if (tid == 0) s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) return;
    if (row >= a.rows) return;
    // merge (same arithmetic as lse_merge_kernel); the local part is read in place
    auto part = [&](int r) -> const float* {
        return r == x.rank ? a.local_part : x.inbox + ((size_t)par * x.world + r) * n;
    };
    float mt = -1e30f;
    for (int r = 0; r < x.world; ++r) mt = fmaxf(mt, __ldcv(part(r) + (size_t)a.rows * a.D + row));
    float w[kMaxPeers], lt = 0.f;
    for (int r = 0; r < x.world; ++r) {
        const float* p = part(r) + (size_t)a.rows * a.D;
        w[r] = __expf(__ldcv(p + row) - mt);
        lt = fmaf(w[r], __ldcv(p + a.rows + row), lt);
    }
    for (int d = tid; d < a.D; d += 128) {
        float o = 0.f;
        for (int r = 0; r < x.world; ++r) o = fmaf(w[r], __ldcv(part(r) + (size_t)row * a.D + d), o);
        a.out[(size_t)row * a.D + d] = lt > 0.f ? o / lt : 0.f;
    }
}

// Low-latency form: every 8-byte inbox element carries its own step number, {value bits, step}.  An
// 8-byte store is one transaction, so a reader that sees the step also sees the value: no fence, no
// separate flag, one NVLink crossing instead of store + acknowledge + flag.  grid = rows CTAs; the CTA of
// a row stores that row (D values, m, l) to every peer, then polls the peers' copies of the same row.
// inbox: uint2 [2][world][n]; zero before the first step (step numbers start at 1).
__global__ void __launch_bounds__(128) exchange_merge_ll_kernel(ExchangeArgs a) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const PeerExchange& x = a.x;
    const unsigned int e = *x.seq;
    const int par = e & 1;
    const size_t n = (size_t)a.rows * (a.D + 2);
    const size_t off_m = (size_t)a.rows * a.D + row, off_l = off_m + a.rows;
    const float my_m = a.local_part[off_m], my_l = a.local_part[off_l];
    for (int r = 0; r < x.world; ++r) {
        if (r == x.rank) continue;
        uint2* dst = reinterpret_cast<uint2*>(x.peer_inbox[r]) + ((size_t)par * x.world + x.rank) * n;
        for (int d = tid; d < a.D; d += 128)
            dst[(size_t)row * a.D + d] = make_uint2(__float_as_uint(a.local_part[(size_t)row * a.D + d]), e);
        if (tid == 0) {
            dst[off_m] = make_uint2(__float_as_uint(my_m), e);
            dst[off_l] = make_uint2(__float_as_uint(my_l), e);
        }
    }
    // All peers are polled side by side: the loads of every missing peer are issued before any is examined, so a
    // round costs one trip to L2 whatever the number of peers.  The arrays are indexed by unrolled constants
    // only and stay in registers.
    const long long t0 = clock64();
    unsigned int peers = 0;
    for (int r = 0; r < x.world; ++r)
        if (r != x.rank) peers |= 1u << r;
    for (int d = tid; d < a.D; d += 128) {
        uint2 vm[kMaxPeers], vl[kMaxPeers], vo[kMaxPeers];
        unsigned int pending = peers;
        bool ok = true;
        while (pending) {
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if (pending >> r & 1u) {
                    const uint2* in = reinterpret_cast<const uint2*>(x.inbox) + ((size_t)par * x.world + r) * n;
                    vm[r] = ld_pair_volatile(in + off_m);
                    vl[r] = ld_pair_volatile(in + off_l);
                    vo[r] = ld_pair_volatile(in + (size_t)row * a.D + d);
                }
#pragma unroll
            for (int r = 0; r < kMaxPeers; ++r)
                if ((pending >> r & 1u) && vm[r].y == e && vl[r].y == e && vo[r].y == e) pending &= ~(1u << r);
            if (pending && clock64() - t0 > x.wait_cycles) {
                ok = false;
                if (a.status && atomicCAS(a.status, 0, GRL_ERR_TIMEOUT) == 0) {
                    a.status[1] = (3 << 28) | (__ffs(pending) - 1);
                    a.status[2] = (int)e;
                    a.status[3] = x.rank;
                }
                break;
            }
        }
        if (!ok) continue;
        float mt = my_m;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (peers >> r & 1u) mt = fmaxf(mt, __uint_as_float(vm[r].x));
        const float w0 = __expf(my_m - mt);
        float o = w0 * a.local_part[(size_t)row * a.D + d], lt = w0 * my_l;
#pragma unroll
        for (int r = 0; r < kMaxPeers; ++r)
            if (peers >> r & 1u) {
                const float w = __expf(__uint_as_float(vm[r].x) - mt);
                o = fmaf(w, __uint_as_float(vo[r].x), o);
                lt = fmaf(w, __uint_as_float(vl[r].x), lt);
            }
        a.out[(size_t)row * a.D + d] = lt > 0.f ? o / lt : 0.f;
    }
}

__global__ void exchange_reset_kernel(uint4* inbox, size_t inbox_vec, unsigned int* flags, size_t n_flags,
                                      unsigned int* seq) {
    const size_t stride = (size_t)gridDim.x * blockDim.x, i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t i = i0; i < inbox_vec; i += stride) inbox[i] = make_uint4(0, 0, 0, 0);
    for (size_t i = i0; i < n_flags; i += stride) flags[i] = 0;
    if (i0 == 0) *seq = 0;
}

}  // namespace grl

using namespace grl;

extern "C" {

int grl_ipc_export(grl_device* dev, void* ptr, void* handle_out) {
    GRL_REQUIRE(dev && ptr && handle_out, "NULL argument");
    DeviceGuard g(dev->ordinal);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    GRL_CUDA(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle_out), ptr));
    return GRL_OK;
}

int grl_ipc_import(grl_device* dev, const void* handle, void** ptr_out) {
    GRL_REQUIRE(dev && handle && ptr_out, "NULL argument");
    DeviceGuard g(dev->ordinal);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    GRL_CUDA(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return GRL_OK;
}

int grl_ipc_release(grl_device* dev, void* ptr) {
    GRL_REQUIRE(dev, "dev is NULL");
    if (!ptr) return GRL_OK;
    DeviceGuard g(dev->ordinal);
    GRL_CUDA(cudaIpcCloseMemHandle(ptr));
    return GRL_OK;
}

int grl_exchange_merge(grl_device* dev, const grl_exchange_params* p) {
    GRL_REQUIRE(dev && p, "NULL argument");
    GRL_REQUIRE(p->rows > 0 && p->head_dim > 0, "bad shape");
    GRL_REQUIRE(p->local_partial && p->out, "NULL buffer");
    GRL_REQUIRE(((uintptr_t)p->local_partial % 16 == 0) && (((size_t)p->rows * (p->head_dim + 2) * 4) % 16 == 0),
                "partials must be 16-byte aligned and a multiple of 16 bytes");
    ExchangeArgs a{};
    int rc = fill_peer_exchange(dev, p, &a.x);
    if (rc) return rc;
    DeviceGuard g(dev->ordinal);
    a.local_part = p->local_partial; a.out = p->out;
    a.status = dev->d_status; a.rows = p->rows; a.D = p->head_dim;
    dev->status_dirty = true;
    bump_seq_kernel<<<1, 1, 0, dev->stream>>>(p->seq);
    GRL_LAUNCHED("bump_seq_kernel");
    if (p->low_latency) {
        exchange_merge_ll_kernel<<<p->rows, 128, 0, dev->stream>>>(a);
        GRL_LAUNCHED("exchange_merge_ll_kernel");
        return GRL_OK;
    }
    const int ctas = p->rows > p->world ? p->rows : p->world;
    exchange_merge_kernel<<<ctas, 128, 0, dev->stream>>>(a);
    GRL_LAUNCHED("exchange_merge_kernel");
    return GRL_OK;
}

int grl_exchange_reset(grl_device* dev, const grl_exchange_params* p) {
    GRL_REQUIRE(dev && p, "NULL argument");
    GRL_REQUIRE(p->inbox && p->flags && p->seq, "NULL buffer");
    GRL_REQUIRE(p->world >= 1 && p->world <= kMaxPeers && p->rows > 0 && p->head_dim > 0, "bad shape");
    GRL_REQUIRE((uintptr_t)p->inbox % 16 == 0, "inbox must be 16-byte aligned");
    DeviceGuard g(dev->ordinal);
    const size_t n = (size_t)p->rows * (p->head_dim + 2);
    const size_t inbox_bytes = 2 * (size_t)p->world * n * (p->low_latency ? 8 : 4);
    const size_t n_flags = 2 * (size_t)p->world * (p->flag_slots > 0 ? p->flag_slots : 1);
    GRL_REQUIRE(inbox_bytes % 16 == 0, "inbox size must be a multiple of 16 bytes");
    exchange_reset_kernel<<<64, 256, 0, dev->stream>>>(reinterpret_cast<uint4*>(p->inbox), inbox_bytes / 16, p->flags,
                                                       n_flags, p->seq);
    GRL_LAUNCHED("exchange_reset_kernel");
    return GRL_OK;
}

}  // extern "C"
