// Halo exchange between neighbouring domains by direct stores into the neighbour GPU's memory.
//
// The role is the one MPI communication plays for the reference when LAMMPS runs it on several ranks
// (ghost positions before PairAI2Pot::compute, reverse communication of the ghost forces after it:
// interface/lammps/AI2POT/pair_ai2pot.cpp:177-205, 452-455). Here the boundary rows are gathered, shifted by the
// periodic image vector where the message wraps around the cell, and written straight into the rows of the
// neighbour's array over NVLink (plain peer stores: no staging buffer, no library call); the last block to finish
// raises a flag in the neighbour's memory with a system-scope release, and the neighbour's next kernels are held
// back by a one-thread wait kernel that polls that flag with system-scope acquires. The wait is bounded: after
// max_polls polls it gives up, records that in a status word and returns, so the context stays usable and the host
// can report AI2B_ERR_TIMEOUT instead of hanging.
//
// A push and the wait for it run on different GPUs (each rank pushes to its neighbours and waits for what they
// push to it), never as two launches on one device that depend on each other.
#include "common.cuh"

namespace ai2b {

template <typename T>
__global__ void peer_push_rows_kernel(const T *__restrict__ src, const int *__restrict__ src_idx, const int *__restrict__ dst_idx, int n,
                                      T sx, T sy, T sz, T *__restrict__ peer_dst, int *peer_flag, int flag_value, unsigned *counter)
{
    for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < n; k += gridDim.x * blockDim.x) {
        const int s = src_idx ? src_idx[k] : k, d = dst_idx ? dst_idx[k] : k;
        const T x = src[3 * (size_t)s] + sx, y = src[3 * (size_t)s + 1] + sy, z = src[3 * (size_t)s + 2] + sz;
        peer_dst[3 * (size_t)d] = x;
        peer_dst[3 * (size_t)d + 1] = y;
        peer_dst[3 * (size_t)d + 2] = z;
    }
    // every thread's stores are ordered before its block's arrival at the counter; the last block to arrive
    // publishes the flag
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned arrived = atomicAdd(counter, 1u);
        if (arrived == gridDim.x - 1) {
            *counter = 0u;                       // ready for the next (stream-ordered) push that uses this counter
            __threadfence_system();
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peer_flag), "r"(flag_value) : "memory");
        }
    }
}

__global__ void peer_wait_kernel(const int *flag, int value, long long max_polls, int *status)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int v = 0;
    long long polls = 0;
    for (;;) {
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= value) break;
        if (++polls >= max_polls) break;
        __nanosleep(200);
    }
    if (v < value) atomicExch(status, 1);        // gave up: the data this wait guards has not arrived
}

// Both directions of one exchange in ONE launch: the blocks split over the two pushes; the last block to arrive
// raises both neighbours' flags and then waits (bounded) for the two flags the neighbours raise here. The
// neighbours' pushes run on their own GPUs and do not depend on this kernel, so the wait cannot deadlock; it gives
// up after max_polls polls and records that in *status.
template <typename T>
struct PeerPush {
    const T *src;
    const int *src_idx, *dst_idx;
    int n;
    T sx, sy, sz;
    T *peer_dst;
    int *peer_flag;
};

template <typename T>
__global__ void peer_exchange_kernel(PeerPush<T> L, PeerPush<T> R, int blocks_left, int flag_value, const int *my_flag_l, const int *my_flag_r,
                                     long long max_polls, int *status, unsigned *counter)
{
    const bool left = (int)blockIdx.x < blocks_left;
    const PeerPush<T> &P = left ? L : R;
    const int b = left ? blockIdx.x : blockIdx.x - blocks_left, nb = left ? blocks_left : gridDim.x - blocks_left;
    for (int k = b * blockDim.x + threadIdx.x; k < P.n; k += nb * blockDim.x) {
        const int s = P.src_idx ? P.src_idx[k] : k, d = P.dst_idx ? P.dst_idx[k] : k;
        const T x = P.src[3 * (size_t)s] + P.sx, y = P.src[3 * (size_t)s + 1] + P.sy, z = P.src[3 * (size_t)s + 2] + P.sz;
        P.peer_dst[3 * (size_t)d] = x;
        P.peer_dst[3 * (size_t)d + 1] = y;
        P.peer_dst[3 * (size_t)d + 2] = z;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x != 0) return;
    const unsigned arrived = atomicAdd(counter, 1u);
    if (arrived != gridDim.x - 1) return;
    *counter = 0u;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(L.peer_flag), "r"(flag_value) : "memory");
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(R.peer_flag), "r"(flag_value) : "memory");
    // what the neighbours send here
    int vl = 0, vr = 0;
    long long polls = 0;
    for (;;) {
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(vl) : "l"(my_flag_l) : "memory");
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(vr) : "l"(my_flag_r) : "memory");
        if (vl >= flag_value && vr >= flag_value) break;
        if (++polls >= max_polls) break;
        __nanosleep(50);
    }
    if (vl < flag_value || vr < flag_value) atomicExch(status, 1);
}

// The closing exchange of a step in one launch: ghost-force rows to the two neighbours, this rank's partial energy
// and virial to every rank, then (after the bounded waits) the neighbours' rows added onto the owned atoms and the
// partials of all ranks summed in rank order (so every rank forms the identical sum).
template <typename T>
struct PeerReduce {
    const T *ev_partial;            // [nev] this rank's partial sums
    T *const *peer_ev;              // [nranks] every rank's table [nranks][PEER_EV_STRIDE] (own entry: local address)
    int *const *peer_ev_flag;       // [nranks] every rank's flag array [nranks]
    const T *my_ev;                 // this rank's table
    const int *my_ev_flag;          // this rank's flag array
    T *ev_out;                      // [nev] the reduced values
    int rank, nranks, nev;
};
constexpr int PEER_EV_STRIDE = 16;

template <typename T>
__global__ void peer_return_reduce_kernel(PeerPush<T> L, PeerPush<T> R, int blocks_left, int flag_value, const int *my_flag_l,
                                          const int *my_flag_r, const T *back, const int *back_idx, int nback, T *force, PeerReduce<T> E,
                                          long long max_polls, int *status, unsigned *counter)
{
    __shared__ int s_ok;
    const bool left = (int)blockIdx.x < blocks_left;
    const PeerPush<T> &P = left ? L : R;
    const int b = left ? blockIdx.x : blockIdx.x - blocks_left, nb = left ? blocks_left : gridDim.x - blocks_left;
    for (int k = b * blockDim.x + threadIdx.x; k < P.n; k += nb * blockDim.x) {
        const T x = P.src[3 * (size_t)k], y = P.src[3 * (size_t)k + 1], z = P.src[3 * (size_t)k + 2];
        P.peer_dst[3 * (size_t)k] = x;
        P.peer_dst[3 * (size_t)k + 1] = y;
        P.peer_dst[3 * (size_t)k + 2] = z;
    }
    __threadfence_system();
    __syncthreads();
    bool last = false;
    if (threadIdx.x == 0) {
        const unsigned arrived = atomicAdd(counter, 1u);
        last = arrived == gridDim.x - 1;
        if (last) {
            __threadfence_system();
            if (L.peer_flag) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(L.peer_flag), "r"(flag_value) : "memory");
            if (R.peer_flag) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(R.peer_flag), "r"(flag_value) : "memory");
        }
        s_ok = last ? 2 : 0;
    }
    __syncthreads();
    const bool is_last = s_ok == 2;
    __syncthreads();        // s_ok is reused below
    // the last block also publishes this rank's partial energy / virial to every rank (own table included)
    if (is_last && E.nranks > 0) {
        for (int i = threadIdx.x; i < E.nranks * E.nev; i += blockDim.x) {
            const int q = i / E.nev, c = i % E.nev;
            E.peer_ev[q][E.rank * PEER_EV_STRIDE + c] = E.ev_partial[c];
        }
        __threadfence_system();
        __syncthreads();
        for (int q = threadIdx.x; q < E.nranks; q += blockDim.x)
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(E.peer_ev_flag[q] + E.rank), "r"(flag_value) : "memory");
    }
    // every block waits for the neighbours' force rows, then adds its share of them onto the owned atoms
    if (nback > 0) {
        if (threadIdx.x == 0) {
            int vl = 0, vr = 0;
            long long polls = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(vl) : "l"(my_flag_l) : "memory");
                asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(vr) : "l"(my_flag_r) : "memory");
                if (vl >= flag_value && vr >= flag_value) break;
                if (++polls >= max_polls) break;
                __nanosleep(50);
            }
            const bool ok = vl >= flag_value && vr >= flag_value;
            if (!ok) atomicExch(status, 1);
            s_ok = ok ? 1 : 0;
        }
        __syncthreads();
        if (s_ok == 1)      // rows are added with atomics: an atom can sit in both send lists of a narrow slab
            for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < nback; k += gridDim.x * blockDim.x) {
                const int i = back_idx[k];
                atomicAdd(force + 3 * (size_t)i, back[3 * (size_t)k]);
                atomicAdd(force + 3 * (size_t)i + 1, back[3 * (size_t)k + 1]);
                atomicAdd(force + 3 * (size_t)i + 2, back[3 * (size_t)k + 2]);
            }
    }
    // the last block collects every rank's partials and sums them in rank order
    if (is_last && E.nranks > 0) {
        __syncthreads();
        if (threadIdx.x < 32) {
            bool ok = true;
            for (int q = threadIdx.x; q < E.nranks; q += 32) {
                int v = 0;
                long long polls = 0;
                for (;;) {
                    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(E.my_ev_flag + q) : "memory");
                    if (v >= flag_value) break;
                    if (++polls >= max_polls) break;
                    __nanosleep(50);
                }
                ok = ok && v >= flag_value;
            }
            ok = __all_sync(FULL_MASK, ok);
            if (!ok && threadIdx.x == 0) atomicExch(status, 1);
            if (ok && (int)threadIdx.x < E.nev) {
                T sum = T(0);
                for (int q = 0; q < E.nranks; q++) sum += E.my_ev[q * PEER_EV_STRIDE + threadIdx.x];
                E.ev_out[threadIdx.x] = sum;
            }
        }
    }
    if (is_last && threadIdx.x == 0) *counter = 0u;
}

template <typename T>
static int peer_return_reduce(const T *src_l, int n_l, T *dst_l, int *flag_l, const T *src_r, int n_r, T *dst_r, int *flag_r, int flag_value,
                              const int *my_flag_l, const int *my_flag_r, const T *back, const int *back_idx, int nback, T *force,
                              const T *ev_partial, T *const *peer_ev, int *const *peer_ev_flag, const T *my_ev, const int *my_ev_flag,
                              T *ev_out, int rank, int nranks, int nev, long long max_polls, int *status, unsigned *counter, cudaStream_t st)
{
    AI2B_REQUIRE(n_l >= 0 && n_r >= 0 && nback >= 0 && max_polls > 0, AI2B_ERR_INVALID, "ai2b_peer_return_reduce: bad count");
    AI2B_REQUIRE(status && counter, AI2B_ERR_INVALID, "ai2b_peer_return_reduce: NULL status or counter");
    AI2B_REQUIRE(nranks >= 0 && nranks <= 1024 && nev >= 0 && nev <= PEER_EV_STRIDE && rank >= 0 && (nranks == 0 || rank < nranks), AI2B_ERR_INVALID,
                 "ai2b_peer_return_reduce: bad rank layout (at most %d values per rank)", PEER_EV_STRIDE);
    AI2B_REQUIRE(nranks == 0 || (ev_partial && peer_ev && peer_ev_flag && my_ev && my_ev_flag && ev_out), AI2B_ERR_INVALID,
                 "ai2b_peer_return_reduce: NULL reduction argument");
    AI2B_REQUIRE((n_l + n_r == 0 && nback == 0) || (flag_l && flag_r && my_flag_l && my_flag_r), AI2B_ERR_INVALID,
                 "ai2b_peer_return_reduce: NULL flag");
    AI2B_REQUIRE((n_l == 0 || (src_l && dst_l)) && (n_r == 0 || (src_r && dst_r)) && (nback == 0 || (back && back_idx && force)), AI2B_ERR_INVALID,
                 "ai2b_peer_return_reduce: NULL argument");
    // without rows to exchange the neighbour flags are not touched: point them at a private dummy is the caller's job
    PeerPush<T> L{src_l, nullptr, nullptr, n_l, T(0), T(0), T(0), dst_l, flag_l};
    PeerPush<T> R{src_r, nullptr, nullptr, n_r, T(0), T(0), T(0), dst_r, flag_r};
    PeerReduce<T> E{ev_partial, peer_ev, peer_ev_flag, my_ev, my_ev_flag, ev_out, rank, nranks, nev};
    auto nblk = [](int n) { int b = (n + 255) / 256; return b < 1 ? 1 : (b > 48 ? 48 : b); };
    const int bl = nblk(n_l), br = nblk(n_r);
    peer_return_reduce_kernel<T><<<bl + br, 256, 0, st>>>(L, R, bl, flag_value, my_flag_l, my_flag_r, back, back_idx, nback, force, E, max_polls,
                                                        status, counter);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

template <typename T>
static int peer_exchange(const T *src_l, const int *sidx_l, const int *didx_l, int n_l, const T *h_shift_l, T *dst_l, int *flag_l,
                         const T *src_r, const int *sidx_r, const int *didx_r, int n_r, const T *h_shift_r, T *dst_r, int *flag_r,
                         int flag_value, const int *my_flag_l, const int *my_flag_r, long long max_polls, int *status, unsigned *counter,
                         cudaStream_t st)
{
    AI2B_REQUIRE(n_l >= 0 && n_r >= 0 && max_polls > 0, AI2B_ERR_INVALID, "ai2b_peer_exchange: bad count");
    AI2B_REQUIRE(flag_l && flag_r && my_flag_l && my_flag_r && status && counter, AI2B_ERR_INVALID, "ai2b_peer_exchange: NULL flag, status or counter");
    AI2B_REQUIRE((n_l == 0 || (src_l && dst_l)) && (n_r == 0 || (src_r && dst_r)), AI2B_ERR_INVALID, "ai2b_peer_exchange: NULL argument");
    PeerPush<T> L{src_l, sidx_l, didx_l, n_l, h_shift_l ? h_shift_l[0] : T(0), h_shift_l ? h_shift_l[1] : T(0), h_shift_l ? h_shift_l[2] : T(0), dst_l, flag_l};
    PeerPush<T> R{src_r, sidx_r, didx_r, n_r, h_shift_r ? h_shift_r[0] : T(0), h_shift_r ? h_shift_r[1] : T(0), h_shift_r ? h_shift_r[2] : T(0), dst_r, flag_r};
    auto nblk = [](int n) { int b = (n + 255) / 256; return b < 1 ? 1 : (b > 48 ? 48 : b); };
    const int bl = nblk(n_l), br = nblk(n_r);
    peer_exchange_kernel<T><<<bl + br, 256, 0, st>>>(L, R, bl, flag_value, my_flag_l, my_flag_r, max_polls, status, counter);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

template <typename T>
static int peer_push_rows(const T *src, const int *src_idx, const int *dst_idx, int n, const T *h_shift3, T *peer_dst, int *peer_flag,
                          int flag_value, unsigned *counter, cudaStream_t st)
{
    AI2B_REQUIRE(n >= 0, AI2B_ERR_INVALID, "ai2b_peer_push_rows: negative row count");
    AI2B_REQUIRE(peer_flag && counter, AI2B_ERR_INVALID, "ai2b_peer_push_rows: NULL flag or counter");
    AI2B_REQUIRE(n == 0 || (src && peer_dst), AI2B_ERR_INVALID, "ai2b_peer_push_rows: NULL argument");
    const T sx = h_shift3 ? h_shift3[0] : T(0), sy = h_shift3 ? h_shift3[1] : T(0), sz = h_shift3 ? h_shift3[2] : T(0);
    int blocks = (n + 255) / 256;
    blocks = blocks < 1 ? 1 : (blocks > 64 ? 64 : blocks);      // a few blocks saturate the link for messages of this size
    peer_push_rows_kernel<T><<<blocks, 256, 0, st>>>(src, src_idx, dst_idx, n, sx, sy, sz, peer_dst, peer_flag, flag_value, counter);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}

}  // namespace ai2b

using namespace ai2b;

extern "C" int ai2b_peer_push_rows_f32(const float *d_src, const int *d_src_index, const int *d_dst_index, int nrows, const float *h_shift3,
                                       float *d_peer_dst, int *d_peer_flag, int flag_value, unsigned *d_counter, void *stream)
{
    return peer_push_rows<float>(d_src, d_src_index, d_dst_index, nrows, h_shift3, d_peer_dst, d_peer_flag, flag_value, d_counter,
                                 (cudaStream_t)stream);
}
extern "C" int ai2b_peer_push_rows_f64(const double *d_src, const int *d_src_index, const int *d_dst_index, int nrows, const double *h_shift3,
                                       double *d_peer_dst, int *d_peer_flag, int flag_value, unsigned *d_counter, void *stream)
{
    return peer_push_rows<double>(d_src, d_src_index, d_dst_index, nrows, h_shift3, d_peer_dst, d_peer_flag, flag_value, d_counter,
                                  (cudaStream_t)stream);
}

#define AI2B_DEF_PEER_EXCHANGE(SUF, T)                                                                                  \
    extern "C" int ai2b_peer_exchange_##SUF(const T *d_src_l, const int *d_src_index_l, const int *d_dst_index_l, int nrows_l,  \
                                            const T *h_shift3_l, T *d_peer_dst_l, int *d_peer_flag_l, const T *d_src_r,        \
                                            const int *d_src_index_r, const int *d_dst_index_r, int nrows_r,                   \
                                            const T *h_shift3_r, T *d_peer_dst_r, int *d_peer_flag_r, int flag_value,          \
                                            const int *d_my_flag_l, const int *d_my_flag_r, long long max_polls, int *d_status, \
                                            unsigned *d_counter, void *stream)                                                  \
    {                                                                                                                           \
        return peer_exchange<T>(d_src_l, d_src_index_l, d_dst_index_l, nrows_l, h_shift3_l, d_peer_dst_l, d_peer_flag_l, d_src_r, \
                                d_src_index_r, d_dst_index_r, nrows_r, h_shift3_r, d_peer_dst_r, d_peer_flag_r, flag_value,     \
                                d_my_flag_l, d_my_flag_r, max_polls, d_status, d_counter, (cudaStream_t)stream);                \
    }
AI2B_DEF_PEER_EXCHANGE(f32, float)
AI2B_DEF_PEER_EXCHANGE(f64, double)

#define AI2B_DEF_PEER_RETURN(SUF, T)                                                                                        \
    extern "C" int ai2b_peer_return_reduce_##SUF(const T *d_src_l, int nrows_l, T *d_peer_dst_l, int *d_peer_flag_l, const T *d_src_r, \
                                                 int nrows_r, T *d_peer_dst_r, int *d_peer_flag_r, int flag_value,                  \
                                                 const int *d_my_flag_l, const int *d_my_flag_r, const T *d_back,                   \
                                                 const int *d_back_index, int nback, T *d_force, const T *d_partial,                \
                                                 T *const *d_peer_tables, int *const *d_peer_table_flags, const T *d_my_table,      \
                                                 const int *d_my_table_flags, T *d_reduced, int rank, int nranks, int nvalues,      \
                                                 long long max_polls, int *d_status, unsigned *d_counter, void *stream)             \
    {                                                                                                                               \
        return peer_return_reduce<T>(d_src_l, nrows_l, d_peer_dst_l, d_peer_flag_l, d_src_r, nrows_r, d_peer_dst_r, d_peer_flag_r,   \
                                     flag_value, d_my_flag_l, d_my_flag_r, d_back, d_back_index, nback, d_force, d_partial,         \
                                     d_peer_tables, d_peer_table_flags, d_my_table, d_my_table_flags, d_reduced, rank, nranks,      \
                                     nvalues, max_polls, d_status, d_counter, (cudaStream_t)stream);                                \
    }
AI2B_DEF_PEER_RETURN(f32, float)
AI2B_DEF_PEER_RETURN(f64, double)

extern "C" int ai2b_peer_wait(const int *d_flag, int value, long long max_polls, int *d_status, void *stream)
{
    AI2B_REQUIRE(d_flag && d_status && max_polls > 0, AI2B_ERR_INVALID, "ai2b_peer_wait: bad argument");
    peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(d_flag, value, max_polls, d_status);
    AI2B_CUDA(cudaGetLastError());
    return AI2B_OK;
}
