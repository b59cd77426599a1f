// Compiled form of the MTP alpha tables, shared by the MTP kernels.
//
// The reference walks alpha_index_basic / alpha_index_times row by row for every atom
// (source/descriptor/mtpr/include/mtpBasis.h:472-528, linearMtp.h:292-306). Here the tables are
// analysed once on the host:
//  * basic moments (mu, ax, ay, az) are mapped onto a dense, degree-major canonical monomial
//    numbering per mu, so the kernels evaluate them with compile-time exponents;
//  * product rows (a, b, mult, dst) are grouped by destination and by dependency depth, so a
//    warp runs all destinations of one depth in parallel (forward), and the adjoint sweep is
//    turned into a gather per source moment (reverse).
#pragma once
#include "common.cuh"

namespace ai2b {

constexpr int MTP_MAX_MU = 8;
constexpr int MTP_MAX_DEG = 8;
constexpr int MTP_MAX_LEV = 16;

struct MtpProgramDev {
    int nm, nb, nt, ns, nmus, kmax, ndense, nlev;
    int kmu[MTP_MAX_MU];            // highest monomial degree used with radial function mu
    int doff[MTP_MAX_MU + 1];       // dense offset of mu: doff[mu] + canonical index
    int fwd_lev_off[MTP_MAX_LEV + 1];  // destinations of depth 1..nlev
    int rev_lev_off[MTP_MAX_LEV + 1];  // source moments of depth nlev-1..0
    const int *basic_dense;         // [nb] dense index of basic row i
    const int *dense_basic;         // [ndense] basic row of dense index d (-1: the tables have no such moment)
    const int4 *e4d;                // [ndense] dense indices holding {value, d/dx, d/dy, d/dz} sources (-1: none)
    const int4 *e4g;                // [ndense] basic row holding {value, d/dx, d/dy, d/dz} source (-1: none)
    const int *e4m;                 // [ndense] packed multipliers (ax+1) | (ay+1)<<8 | (az+1)<<16
    const int4 *fwd_dst;            // {dst, row_begin, row_end, -}
    const int *fwd_ab;              // [nt] a | b<<16, rows grouped by destination
    const float *fwd_mult_f;        // [nt] multiplier, float / double copies (no int->fp conversion on the device)
    const double *fwd_mult_d;
    const int2 *fwd_rows;           // [nt] {a | b<<16, multiplier as float bits}: one 8-byte load per row
    const int2 *rev_ents;           // [2 nt] {other | dst<<16, multiplier as float bits}
    // flat row streams for the lanes-as-atoms kernel: rows of one depth are contiguous, a flag marks the
    // last row of each destination, so any contiguous share of a depth's rows can be given to a worker
    const int2 *fwd_flat;           // [nt]   {a | b<<16, mult | last<<8 | dst<<16}
    const int2 *rev_flat;           // [2 nt] {other | dst<<16, mult | last<<8 | source<<16}
    int fwd_lev_row[MTP_MAX_LEV + 1];
    int rev_lev_row[MTP_MAX_LEV + 1];
    const int4 *rev_mom;            // {m, entry_begin, entry_end, -}
    const int *rev_od;              // [2 nt] other | dst<<16
    const float *rev_mult_f;
    const double *rev_mult_d;
    const int *map;                 // [ns] alpha_moment_mapping
    // Segment streams of the lanes-as-atoms contraction (tiles of MTP_TILE atoms, MTP_SEG_WORKERS workers):
    // the rows that feed one moment with one multiplier form a segment {header, rows}. Phase p < nlev is
    // product depth p + 1 (rows {a, b}: M[dst] = sum mult * M[a] * M[b]); phase nlev + k gathers the adjoints
    // of the source moments of depth nlev - 1 - k (rows {dst, other}: E[src] = seed + sum mult * E[dst] * M[other]).
    // Every moment's segments belong to ONE worker and are consecutive, so there are no atomics; the
    // moments of a phase are dealt to the workers by decreasing row count (longest processing time first).
    // All moment references are element offsets m * MTP_SEG_LD.
    const int4 *seg_hdr;            // [nseg] {moment offset, nrows | first << 30 | last << 31, multiplier (double) lo, hi}
    const int2 *seg_row;            // [2 nt rows of the adjoint phases + nt of the product phases]
    const int *seg_wseg;            // [2 nlev][MTP_SEG_WORKERS + 1] first header of worker w in phase p
    const int *seg_wrow;            // [2 nlev][MTP_SEG_WORKERS] first row of worker w in phase p
    const int *seg_init;            // [nseg_init] moments whose adjoint is only their seed (no product reads them)
    int nseg, nseg_rows, nseg_init;
};
constexpr int MTP_SEG_WORKERS = 32;
constexpr int MTP_TILE = 32;        // atoms per tile of the contraction
constexpr int MTP_SEG_LD = 33;      // row stride of its [moment][atom] arrays

template <typename T> __device__ __forceinline__ const T *fwd_mult(const MtpProgramDev &P);
template <> __device__ __forceinline__ const float *fwd_mult<float>(const MtpProgramDev &P) { return P.fwd_mult_f; }
template <> __device__ __forceinline__ const double *fwd_mult<double>(const MtpProgramDev &P) { return P.fwd_mult_d; }
template <typename T> __device__ __forceinline__ const T *rev_mult(const MtpProgramDev &P);
template <> __device__ __forceinline__ const float *rev_mult<float>(const MtpProgramDev &P) { return P.rev_mult_f; }
template <> __device__ __forceinline__ const double *rev_mult<double>(const MtpProgramDev &P) { return P.rev_mult_d; }

}  // namespace ai2b

struct ai2b_mtp_program {
    ai2b::MtpProgramDev dev;
    void *d_blob;       // one device allocation holding every table
    size_t blob_bytes;
    int device;
};
