// Neighbour rows of a tile of 32 atoms in shared memory, for the kernels whose lanes are atoms.
//
// With one atom per lane every lane walks along its own row of the padded neighbour arrays
// (rcs[slot][umax][3], firstneigh[slot][umax]), so a warp's load touches 32 different rows: 32 sectors per
// instruction, and a dependent index -> type look-up behind it. Here the block copies the first
// TR_SLOTS slots of its 32 rows with loads that run ALONG the rows (consecutive threads read consecutive
// elements), all of them in flight together, and the lanes then read their row from shared memory:
//   pos[atom][TR_RS]   r_j - r_i of slots 0 .. TR_SLOTS-1 (row stride odd: the 32 rows start in different banks)
//   idx[atom][TR_IS]   neighbour index | neighbour type << 26 (0 for empty slots)
// Slots beyond TR_SLOTS (rows longer than 32 neighbours) are read from global memory by the caller.
#pragma once
#include <cuda_pipeline.h>
#include "common.cuh"

namespace ai2b {

constexpr int TR_SLOTS = 32;
constexpr int TR_RS = 3 * TR_SLOTS + 1;
constexpr int TR_IS = TR_SLOTS + 1;
constexpr int TR_TYPE_SHIFT = 26;                 // atom indices below 2^26, types below 32
constexpr int TR_INDEX_MASK = (1 << TR_TYPE_SHIFT) - 1;

template <typename T>
__host__ __device__ constexpr size_t tile_rows_bytes()
{
    return ((sizeof(T) * 32 * TR_RS + 15) & ~size_t(15)) + 2 * sizeof(int) * 32 * TR_IS + 32 * (2 * sizeof(long long) + sizeof(int)) + 16;
}

template <typename T>
struct TileRows {
    T *pos;
    int *idx;
    long long *row;     // [32] first slot of the atom's row in the neighbour arrays (atom slot * umax)
    long long *tbase;   // [32] offset of the atom's structure in the type array
    int *nn;            // [32] neighbours of the atom (clamped to umax)
    int *raw;           // [32][TR_IS] neighbour indices as copied, before their types are looked up (single-structure path)

    __device__ __forceinline__ void bind(unsigned char *mem)
    {
        pos = reinterpret_cast<T *>(mem);
        unsigned char *p = mem + ((sizeof(T) * 32 * TR_RS + 15) & ~size_t(15));
        row = reinterpret_cast<long long *>(p);
        tbase = row + 32;
        idx = reinterpret_cast<int *>(tbase + 32);
        nn = idx + 32 * TR_IS;
        raw = nn + 32;
    }
    // one warp, lane = atom of the tile
    __device__ __forceinline__ void describe(int lane, size_t first_slot, size_t types_offset, int count)
    {
        row[lane] = (long long)first_slot;
        tbase[lane] = (long long)types_offset;
        nn[lane] = count;
    }
    // all NT threads of the block, after a barrier behind describe(); a barrier must follow
    template <int NT>
    __device__ __forceinline__ void stage(const T *__restrict__ rcs, const int *__restrict__ firstneigh, const int *__restrict__ types,
                                          int umax)
    {
        const int lim = 3 * (umax < TR_SLOTS ? umax : TR_SLOTS);
        constexpr int TP = 32 * 3 * TR_SLOTS, TI = 32 * TR_SLOTS;           // elements of the two copies
        constexpr int NP = (TP + NT - 1) / NT, NI = (TI + NT - 1) / NT;     // per thread
        T v[NP];
        int nj[NI], w[NI];
#pragma unroll
        for (int k = 0; k < NI; k++) {
            const int e = threadIdx.x + k * NT, a = (e >> 5) & 31, j = e & 31;
            nj[k] = (e < TI && j < nn[a]) ? firstneigh[row[a] + j] : -1;
        }
#pragma unroll
        for (int k = 0; k < NP; k++) {
            const int e = threadIdx.x + k * NT, a = (e / (3 * TR_SLOTS)) & 31, o = e % (3 * TR_SLOTS);
            v[k] = (e < TP && o < lim) ? rcs[row[a] * 3 + o] : T(0);
        }
#pragma unroll
        for (int k = 0; k < NI; k++) {
            const int e = threadIdx.x + k * NT, a = (e >> 5) & 31;
            w[k] = nj[k] >= 0 ? (nj[k] | (types[tbase[a] + nj[k]] << TR_TYPE_SHIFT)) : 0;
        }
#pragma unroll
        for (int k = 0; k < NP; k++) {
            const int e = threadIdx.x + k * NT, a = e / (3 * TR_SLOTS), o = e % (3 * TR_SLOTS);
            if (e < TP) pos[a * TR_RS + o] = v[k];
        }
#pragma unroll
        for (int k = 0; k < NI; k++) {
            const int e = threadIdx.x + k * NT, a = e >> 5, j = e & 31;
            if (e < TI) idx[a * TR_IS + j] = w[k];
        }
    }

    // Single structure: atom a of the tile is slot first_slot + a, so its rows can be requested before anything about the
    // atoms has been looked up. request() issues asynchronous copies straight into shared memory (no registers are held
    // while the caller does its look-ups); complete(), after the caller's __pipeline_wait_prior(0) and a barrier, looks up
    // the neighbours' types. Slots whose index is outside [0, ids) are empty (rows are padded with -1). Both are called
    // by all NT threads; a barrier must follow complete().
    template <int NT>
    __device__ __forceinline__ void request(const T *__restrict__ rcs, const int *__restrict__ firstneigh, int umax, size_t first_slot,
                                            size_t nslots)
    {
        const int lim = umax < TR_SLOTS ? umax : TR_SLOTS;
        for (int e = threadIdx.x; e < 32 * 3 * TR_SLOTS; e += NT) {
            const int a = e / (3 * TR_SLOTS), o = e % (3 * TR_SLOTS);
            if (o < 3 * lim && first_slot + a < nslots) __pipeline_memcpy_async(pos + a * TR_RS + o, rcs + (first_slot + a) * umax * 3 + o, sizeof(T));
        }
        for (int e = threadIdx.x; e < 32 * TR_SLOTS; e += NT) {
            const int a = e >> 5, j = e & 31;
            if (j < lim && first_slot + a < nslots) __pipeline_memcpy_async(raw + a * TR_IS + j, firstneigh + (first_slot + a) * umax + j, sizeof(int));
            else raw[a * TR_IS + j] = -1;
        }
        __pipeline_commit();
    }
    template <int NT>
    __device__ __forceinline__ void complete(const int *__restrict__ types, int ids)
    {
        constexpr int NI = (32 * TR_SLOTS + NT - 1) / NT;
        int nj[NI], w[NI];
#pragma unroll
        for (int k = 0; k < NI; k++) {
            const int e = threadIdx.x + k * NT;
            nj[k] = e < 32 * TR_SLOTS ? raw[(e >> 5) * TR_IS + (e & 31)] : -1;
        }
#pragma unroll
        for (int k = 0; k < NI; k++) w[k] = (nj[k] >= 0 && nj[k] < ids) ? (nj[k] | (types[nj[k]] << TR_TYPE_SHIFT)) : 0;
#pragma unroll
        for (int k = 0; k < NI; k++) {
            const int e = threadIdx.x + k * NT;
            if (e < 32 * TR_SLOTS) idx[(e >> 5) * TR_IS + (e & 31)] = w[k];
        }
    }
};

}  // namespace ai2b
