/* TEST INFRASTRUCTURE — plain-C restatement of the reference CPU algorithms, one copy per
 * float type (included twice by oracle.c with T / SUF defined). Not shipped, never on the
 * product path. Paths cited are relative to the reference project root. */

/* ---------------------------------------------------------------------------------------
 * Neighbour list. Follows source/nblist/include/structure.h:589-710 (periodic images, image
 * position = ((r + a0*ix) + a1*iy) + a2*iz, loop order ix, iy, iz, atom),
 * binLinkedList.h:658-696 (image range e_k = ceil(rcut/d_k) on periodic axes) and :983-1031
 * (membership: 1e-3 < d2 < rcut^2, squares through pow(x,2), which promotes float to double),
 * neighborList.h:532-578 (index % inum, rcs = r_image - r_centre, padding -1 / 0).
 * Candidate search here is a uniform grid over the images; only the membership predicate and
 * the rcs bits are part of the contract, the order is not (unless sort != 0).
 * ------------------------------------------------------------------------------------- */
static void NAME(cross)(const T *a, const T *b, T *c)
{
    c[0] = a[1] * b[2] - a[2] * b[1];
    c[1] = a[2] * b[0] - a[0] * b[2];
    c[2] = a[0] * b[1] - a[1] * b[0];
}

/* interplanar distances: structure.h:818-843 with core/include/vec3Operation.h cross/normalize/dot */
static void NAME(plane_dist)(const T *cell, T *d)
{
    for (int k = 0; k < 3; k++) {
        const T *o1 = cell + 3 * ((k == 0) ? 1 : 0);
        const T *o2 = cell + 3 * ((k == 2) ? 1 : 2);
        T n[3];
        NAME(cross)(o1, o2, n);
        T len = (T)sqrt((double)(n[0] * n[0] + n[1] * n[1] + n[2] * n[2]));
        T u[3] = {n[0] / len, n[1] / len, n[2] / len};
        const T *a = cell + 3 * k;
        T dot = a[0] * u[0] + a[1] * u[1] + a[2] * u[2];
        d[k] = (T)fabs((double)dot);
    }
}

typedef struct { T d; int idx; T r[3]; } NAME(nbr);
static int NAME(cmp_nbr)(const void *a, const void *b)
{
    T x = ((const NAME(nbr) *)a)->d, y = ((const NAME(nbr) *)b)->d;
    return (x > y) - (x < y);
}

int NAME2(orc_nblist)(int n, const T *cell, const int *types, const T *coords_in, int is_cart,
                      double rcut_d, const int *pbc, int sort, int umax, int *numneigh,
                      int *firstneigh, T *rcs, int *types_out, int *max_nn)
{
    T rcut = (T)rcut_d;
    T *pos = (T *)malloc(sizeof(T) * 3 * (size_t)n);
    for (int i = 0; i < n; i++)
        for (int c = 0; c < 3; c++)
            pos[3 * i + c] = is_cart ? coords_in[3 * i + c]
                                     : (coords_in[3 * i + 0] * cell[0 + c] + coords_in[3 * i + 1] * cell[3 + c]
                                        + coords_in[3 * i + 2] * cell[6 + c]);   /* structure.h:561-581 */
    T dpl[3];
    NAME(plane_dist)(cell, dpl);
    int e[3];
    for (int k = 0; k < 3; k++) e[k] = pbc[k] ? (int)ceil((double)(rcut / dpl[k])) : 0;
    int nim = (2 * e[0] + 1) * (2 * e[1] + 1) * (2 * e[2] + 1);
    size_t ntot = (size_t)nim * n;
    T *img = (T *)malloc(sizeof(T) * 3 * ntot);
    size_t q = 0;
    for (int ix = -e[0]; ix <= e[0]; ix++)
        for (int iy = -e[1]; iy <= e[1]; iy++)
            for (int iz = -e[2]; iz <= e[2]; iz++)
                for (int a = 0; a < n; a++, q++)
                    for (int c = 0; c < 3; c++)
                        img[3 * q + c] = pos[3 * a + c] + cell[0 + c] * (T)ix + cell[3 + c] * (T)iy + cell[6 + c] * (T)iz;
    /* uniform grid over all images, cell edge >= rcut */
    double lo[3] = {1e300, 1e300, 1e300}, hi[3] = {-1e300, -1e300, -1e300};
    for (size_t i = 0; i < ntot; i++)
        for (int c = 0; c < 3; c++) {
            if (img[3 * i + c] < lo[c]) lo[c] = img[3 * i + c];
            if (img[3 * i + c] > hi[c]) hi[c] = img[3 * i + c];
        }
    int ng[3];
    double gs = (double)rcut * 1.0001;
    for (int c = 0; c < 3; c++) { ng[c] = (int)((hi[c] - lo[c]) / gs) + 1; }
    size_t ncell = (size_t)ng[0] * ng[1] * ng[2];
    int *head = (int *)malloc(sizeof(int) * ncell), *next = (int *)malloc(sizeof(int) * ntot);
    for (size_t i = 0; i < ncell; i++) head[i] = -1;
    for (size_t i = 0; i < ntot; i++) {
        int g[3];
        for (int c = 0; c < 3; c++) { g[c] = (int)((img[3 * i + c] - lo[c]) / gs); if (g[c] >= ng[c]) g[c] = ng[c] - 1; }
        size_t ci = ((size_t)g[0] * ng[1] + g[1]) * ng[2] + g[2];
        next[i] = head[ci]; head[ci] = (int)i;
    }
    double rc2 = pow((double)rcut, 2);   /* pow(T,int) promotes to double (binLinkedList.h:1014) */
    int mx = 0, overflow = 0;
    size_t centre0 = (size_t)((e[0] * (2 * e[1] + 1) + e[1]) * (2 * e[2] + 1) + e[2]) * n;
    NAME(nbr) *buf = (NAME(nbr) *)malloc(sizeof(NAME(nbr)) * 4096);
    int bufcap = 4096;
    if (numneigh) {
        for (size_t i = 0; i < (size_t)n * umax; i++) firstneigh[i] = -1;
        memset(rcs, 0, sizeof(T) * 3 * (size_t)n * umax);
    }
    for (int i = 0; i < n; i++) {
        const T *rc_ = img + 3 * (centre0 + i);
        int g[3], cnt = 0;
        for (int c = 0; c < 3; c++) { g[c] = (int)((rc_[c] - lo[c]) / gs); if (g[c] >= ng[c]) g[c] = ng[c] - 1; }
        for (int dx = -1; dx <= 1; dx++) for (int dy = -1; dy <= 1; dy++) for (int dz = -1; dz <= 1; dz++) {
            int x = g[0] + dx, y = g[1] + dy, z = g[2] + dz;
            if (x < 0 || y < 0 || z < 0 || x >= ng[0] || y >= ng[1] || z >= ng[2]) continue;
            for (int j = head[((size_t)x * ng[1] + y) * ng[2] + z]; j != -1; j = next[j]) {
                T d0 = img[3 * (size_t)j + 0] - rc_[0], d1 = img[3 * (size_t)j + 1] - rc_[1], d2 = img[3 * (size_t)j + 2] - rc_[2];
                T dd = (T)((double)d0 * (double)d0 + (double)d1 * (double)d1 + (double)d2 * (double)d2);
                if ((double)dd < rc2 && (double)dd > 1e-3) {
                    if (cnt == bufcap) { bufcap *= 2; buf = (NAME(nbr) *)realloc(buf, sizeof(NAME(nbr)) * bufcap); }
                    buf[cnt].idx = j % n; buf[cnt].r[0] = d0; buf[cnt].r[1] = d1; buf[cnt].r[2] = d2;
                    buf[cnt].d = (T)sqrt((double)d0 * (double)d0 + (double)d1 * (double)d1 + (double)d2 * (double)d2);
                    cnt++;
                }
            }
        }
        if (cnt > mx) mx = cnt;
        if (!numneigh) continue;
        if (cnt > umax) { overflow = 1; continue; }
        if (sort) qsort(buf, cnt, sizeof(NAME(nbr)), NAME(cmp_nbr));
        numneigh[i] = cnt;
        types_out[i] = types[i];
        for (int k = 0; k < cnt; k++) {
            firstneigh[(size_t)i * umax + k] = buf[k].idx;
            for (int c = 0; c < 3; c++) rcs[((size_t)i * umax + k) * 3 + c] = buf[k].r[c];
        }
    }
    if (max_nn) *max_nn = mx;
    free(pos); free(img); free(head); free(next); free(buf);
    return overflow ? -1 : 0;
}

/* ---------------------------------------------------------------------------------------
 * Linear MTP. Radial functions: descriptor/mtpr/include/basis.h:155-181 (quintic switch),
 * :352-380 (Chebyshev value/derivative recurrences), :621-637 (Q = s*T, Q' = s'T + sT').
 * ------------------------------------------------------------------------------------- */
static void NAME(mtp_radial)(T r, T rmax, T rmin, int cs, T *q, T *dq)
{
    T w = (r - rmin) / (rmax - rmin), s = 0, ds = 0;
    if (r >= rmin && r < rmax) {
        s = w * w * w * (-6 * w * w + 15 * w - 10) + 1;
        ds = 1 / (rmax - rmin) * (-30 * w * w * w * w + 60 * w * w * w - 30 * w * w);
    }
    T u = (2 * r - (rmax + rmin)) / (rmax - rmin), uc = 2 / (rmax - rmin);
    T t0 = 1, t1 = u, d0 = 0, d1 = 1;
    for (int k = 0; k < cs; k++) {
        T t, d;
        if (k == 0) { t = 1; d = 0; }
        else if (k == 1) { t = u; d = 1; }
        else { t = 2 * u * t1 - t0; d = 2 * t1 + 2 * u * d1 - d0; t0 = t1; t1 = t; d0 = d1; d1 = d; }
        q[k] = s * t;
        dq[k] = ds * t + s * (d * uc);
    }
}

/* Everything one centre atom needs: moments, and (optionally) per-pair gradients of the basic
 * moments. descriptor/mtpr/include/mtpBasis.h:400-534. `mder` is [nb][nn][3] or NULL. */
typedef struct {
    int cs, nm, nb, nt, ns, nmus, ntypes;
    const int *basic, *times, *map;
    T scaling, rmax, rmin;
    const T *coeffs;
} NAME(mtpdef);

static void NAME(mtp_moments)(const NAME(mtpdef) *m, int ti, int nn, const int *fn, const T *rc,
                              const int *types, T *mom, T *mder)
{
    T q[64], dq[64], pw[3][16], dist_pw[16];
    memset(mom, 0, sizeof(T) * m->nm);
    if (mder) memset(mder, 0, sizeof(T) * 3 * (size_t)m->nb * nn);
    int kmax = 0;
    for (int i = 0; i < m->nb; i++) { int k = m->basic[4 * i + 1] + m->basic[4 * i + 2] + m->basic[4 * i + 3]; if (k > kmax) kmax = k; }
    for (int j = 0; j < nn; j++) {
        const T *v = rc + 3 * j;
        T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
        if (r > m->rmax) continue;
        int tj = types[fn[j]];
        T rinv = 1 / r;
        NAME(mtp_radial)(r, m->rmax, m->rmin, m->cs, q, dq);
        dist_pw[0] = 1; pw[0][0] = pw[1][0] = pw[2][0] = 1;
        for (int k = 1; k <= kmax; k++) {
            dist_pw[k] = dist_pw[k - 1] * r;
            for (int c = 0; c < 3; c++) pw[c][k] = pw[c][k - 1] * v[c];
        }
        for (int i = 0; i < m->nb; i++) {
            const int *al = m->basic + 4 * i;
            int mu = al[0], k = al[1] + al[2] + al[3];
            T C = 1 / dist_pw[k];
            T B = pw[0][al[1]] * pw[1][al[2]] * pw[2][al[3]];
            T Bd[3] = {0, 0, 0};
            if (al[1]) Bd[0] = al[1] * pw[0][al[1] - 1] * pw[1][al[2]] * pw[2][al[3]];
            if (al[2]) Bd[1] = al[2] * pw[0][al[1]] * pw[1][al[2] - 1] * pw[2][al[3]];
            if (al[3]) Bd[2] = al[3] * pw[0][al[1]] * pw[1][al[2]] * pw[2][al[3] - 1];
            const T *co = m->coeffs + ((size_t)(ti * m->ntypes + tj) * m->nmus + mu) * m->cs;
            for (int xi = 0; xi < m->cs; xi++) {
                T A = q[xi] * m->scaling, Ad = dq[xi] * m->scaling;
                mom[i] += co[xi] * A * B * C;
                if (mder)
                    for (int a = 0; a < 3; a++) {
                        T Cd = -k * C * rinv * rinv * v[a];
                        mder[((size_t)i * nn + j) * 3 + a] += co[xi] * (Ad * v[a] * rinv * B * C + A * Bd[a] * C + A * B * Cd);
                    }
            }
        }
    }
    for (int t = 0; t < m->nt; t++) {
        const int *row = m->times + 4 * t;
        mom[row[3]] += (T)row[2] * mom[row[0]] * mom[row[1]];
    }
}

/* adjoint of the site energy w.r.t. every moment: linearMtp.h:292-306 */
static void NAME(mtp_adjoint)(const NAME(mtpdef) *m, const T *mom, const T *lin, const T *qs, T *adj)
{
    memset(adj, 0, sizeof(T) * m->nm);
    for (int s = 0; s < m->ns; s++) adj[m->map[s]] = lin[s] / qs[s];
    for (int t = m->nt - 1; t >= 0; t--) {
        const int *row = m->times + 4 * t;
        adj[row[1]] += adj[row[3]] * (T)row[2] * mom[row[0]];
        adj[row[0]] += adj[row[3]] * (T)row[2] * mom[row[1]];
    }
}

#define NB_DECL int B, int npad, const int *binum, const int *bilist, const int *bnumneigh, \
    const int *bfirstneigh, const T *brcs, const int *btypes, int ntypes, const int *type_map, int umax, int nghost
#define TAB_DECL int nm, int nb, const int *basic, int nt, const int *times, int ns, const int *map, int nmus

/* linearMtp.h:190-352 (efv), :356-510 (ef); batch loop linearMtp_cpu_launcher.h:128-203 */
static void NAME(mtp_efv_impl)(T *betot, T *bforce, T *bvirial, int cs, T scaling, const T *coeffs,
                               const T *lin, const T *bias, TAB_DECL, NB_DECL, T rmax, T rmin, const T *qs)
{
    (void)type_map;
    NAME(mtpdef) m = {cs, nm, nb, nt, ns, nmus, ntypes, basic, times, map, scaling, rmax, rmin, coeffs};
    T *mom = (T *)malloc(sizeof(T) * nm), *adj = (T *)malloc(sizeof(T) * nm);
    T *mder = (T *)malloc(sizeof(T) * 3 * (size_t)nb * umax);
    for (int b = 0; b < B; b++) {
        T *force = bforce + (size_t)b * (npad + nghost) * 3;
        const int *types = btypes + (size_t)b * (npad + nghost);
        T etot = 0, vir[9] = {0};
        memset(force, 0, sizeof(T) * 3 * (size_t)(binum[b] + nghost));
        for (int ii = 0; ii < binum[b]; ii++) {
            size_t slot = (size_t)b * npad + ii;
            int ci = bilist[slot], nn = bnumneigh[slot];
            const int *fn = bfirstneigh + slot * umax;
            const T *rc = brcs + slot * umax * 3;
            NAME(mtp_moments)(&m, types[ci], nn, fn, rc, types, mom, mder);
            T es = bias[types[ci]];
            for (int s = 0; s < ns; s++) es += lin[s] * mom[map[s]] / qs[s];
            etot += es;
            NAME(mtp_adjoint)(&m, mom, lin, qs, adj);
            for (int j = 0; j < nn; j++) {
                const T *v = rc + 3 * j;
                T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
                if (r > rmax) continue;
                for (int a = 0; a < 3; a++) {
                    T g = 0;
                    for (int i = 0; i < nb; i++) g += adj[i] * mder[((size_t)i * nn + j) * 3 + a];
                    force[3 * ci + a] += g;
                    force[3 * fn[j] + a] -= g;
                    for (int c = 0; c < 3; c++) vir[3 * a + c] -= g * v[c];
                }
            }
        }
        betot[b] = etot;
        if (bvirial) memcpy(bvirial + 9 * b, vir, sizeof(vir));
    }
    free(mom); free(adj); free(mder);
}

int NAME2(orc_mtp_efv)(T *betot, T *bforce, T *bvirial, int cs, T scaling, const T *coeffs, const T *lin,
                       const T *bias, TAB_DECL, NB_DECL, T rmax, T rmin, const T *qs)
{
    NAME(mtp_efv_impl)(betot, bforce, bvirial, cs, scaling, coeffs, lin, bias, nm, nb, basic, nt, times, ns, map, nmus,
                       B, npad, binum, bilist, bnumneigh, bfirstneigh, brcs, btypes, ntypes, type_map, umax, nghost, rmax, rmin, qs);
    return 0;
}
int NAME2(orc_mtp_ef)(T *betot, T *bforce, int cs, T scaling, const T *coeffs, const T *lin, const T *bias,
                      TAB_DECL, NB_DECL, T rmax, T rmin, const T *qs)
{
    NAME(mtp_efv_impl)(betot, bforce, NULL, cs, scaling, coeffs, lin, bias, nm, nb, basic, nt, times, ns, map, nmus,
                       B, npad, binum, bilist, bnumneigh, bfirstneigh, brcs, btypes, ntypes, type_map, umax, nghost, rmax, rmin, qs);
    return 0;
}
/* scalar basis values [B, npad, ns], not divided by q_scaler: linearMtp.h find_descriptors,
 * batch loop linearMtp_cpu_launcher.h:284-345 (types row stride is npad there) */
int NAME2(orc_mtp_descriptors)(T *bdesc, int cs, T scaling, const T *coeffs, TAB_DECL, NB_DECL, T rmax, T rmin)
{
    (void)type_map; (void)nghost;
    NAME(mtpdef) m = {cs, nm, nb, nt, ns, nmus, ntypes, basic, times, map, scaling, rmax, rmin, coeffs};
    T *mom = (T *)malloc(sizeof(T) * nm);
    for (int b = 0; b < B; b++) {
        const int *types = btypes + (size_t)b * npad;
        for (int ii = 0; ii < binum[b]; ii++) {
            size_t slot = (size_t)b * npad + ii;
            NAME(mtp_moments)(&m, types[bilist[slot]], bnumneigh[slot], bfirstneigh + slot * umax, brcs + slot * umax * 3, types, mom, NULL);
            for (int s = 0; s < ns; s++) bdesc[slot * ns + s] = mom[map[s]];
        }
    }
    free(mom);
    return 0;
}

/* loss: linearMtpLoss.h:138-210; batch loop linearMtpLoss_cpu_launcher.h:152-231 */
int NAME2(orc_mtp_loss)(T *bloss, int B, int npad, const int *binum, const int *bilist, T ew, T fw, T vw,
                        const T *e_ml, const T *e_dft, const T *f_ml, const T *f_dft, const T *v_ml, const T *v_dft)
{
    for (int b = 0; b < B; b++) {
        int n = binum[b];
        T fl = 0, vl = 0;
        for (int ii = 0; ii < n; ii++) {
            int ci = bilist[(size_t)b * npad + ii];
            for (int a = 0; a < 3; a++) { T d = f_ml[((size_t)b * npad + ci) * 3 + a] - f_dft[((size_t)b * npad + ci) * 3 + a]; fl += d * d; }
        }
        fl = fw / (3 * n) * fl;
        if (v_ml) { for (int k = 0; k < 9; k++) { T d = v_ml[9 * b + k] - v_dft[9 * b + k]; vl += d * d; } vl = vw / (9 * n) * vl; }
        T de = e_ml[b] - e_dft[b];
        bloss[b] = fl + vl + ew / n * de * de;
    }
    return 0;
}
int NAME2(orc_mtp_ef_loss)(T *bloss, int B, int npad, const int *binum, const int *bilist, T ew, T fw,
                           const T *e_ml, const T *e_dft, const T *f_ml, const T *f_dft)
{
    return NAME2(orc_mtp_loss)(bloss, B, npad, binum, bilist, ew, fw, 0, e_ml, e_dft, f_ml, f_dft, NULL, NULL);
}

/* analytic gradient of the loss w.r.t. coeffs, linear_coeffs, type_bias, per structure:
 * linearMtpLoss.h:212-569; batch loop linearMtpLoss_cpu_launcher.h:233-338. Outputs are
 * accumulated into (the caller zeroes them). v_ml == NULL gives the energy+force variant. */
int NAME2(orc_mtp_loss_backward)(T *dco, T *dli, T *dbi, T ew, T fw, T vw, const T *e_ml, const T *e_dft,
                                 const T *f_ml, const T *f_dft, const T *v_ml, const T *v_dft, int cs, T scaling,
                                 const T *coeffs, const T *lin, const T *bias, TAB_DECL, NB_DECL, T rmax, T rmin, const T *qs)
{
    (void)type_map; (void)bias;
    NAME(mtpdef) m = {cs, nm, nb, nt, ns, nmus, ntypes, basic, times, map, scaling, rmax, rmin, coeffs};
    int ncoef = ntypes * ntypes * nmus * cs;
    T *mom = (T *)malloc(sizeof(T) * nm), *adj = (T *)malloc(sizeof(T) * nm), *D = (T *)malloc(sizeof(T) * nm), *G = (T *)malloc(sizeof(T) * nm);
    T *mder = (T *)malloc(sizeof(T) * 3 * (size_t)nb * umax);
    T q[64], dq[64], pw[3][16], dist_pw[16];
    int kmax = 0;
    for (int i = 0; i < nb; i++) { int k = basic[4 * i + 1] + basic[4 * i + 2] + basic[4 * i + 3]; if (k > kmax) kmax = k; }
    for (int b = 0; b < B; b++) {
        int n = binum[b];
        const int *types = btypes + (size_t)b * (npad + nghost);
        const T *fm = f_ml + (size_t)b * npad * 3, *fd = f_dft + (size_t)b * npad * 3;
        T dE = e_ml[b] - e_dft[b], ce = 2 * ew / n * dE, cf = 2 * fw / (3 * n), cv = v_ml ? 2 * vw / (9 * n) : 0;
        T dV[9] = {0};
        if (v_ml) for (int k = 0; k < 9; k++) dV[k] = v_ml[9 * b + k] - v_dft[9 * b + k];
        T *gco = dco + (size_t)b * ncoef, *gli = dli + (size_t)b * ns, *gbi = dbi + (size_t)b * ntypes;
        for (int ii = 0; ii < n; ii++) {
            size_t slot = (size_t)b * npad + ii;
            int ci = bilist[slot], nn = bnumneigh[slot], ti = types[ci];
            const int *fn = bfirstneigh + slot * umax;
            const T *rc = brcs + slot * umax * 3;
            NAME(mtp_moments)(&m, ti, nn, fn, rc, types, mom, mder);
            /* redo the products while carrying the directional derivative D (forward mode) */
            memset(D, 0, sizeof(T) * nm); memset(G, 0, sizeof(T) * nm);
            for (int j = 0; j < nn; j++) {
                const T *v = rc + 3 * j;
                T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
                if (r > rmax) continue;
                for (int a = 0; a < 3; a++) {
                    T p = cf * (fm[3 * ci + a] - fd[3 * ci + a]) - cf * (fm[3 * fn[j] + a] - fd[3 * fn[j] + a]);
                    for (int c = 0; c < 3; c++) p -= cv * dV[3 * a + c] * v[c];
                    for (int i = 0; i < nb; i++) D[i] += p * mder[((size_t)i * nn + j) * 3 + a];
                }
            }
            /* mom currently holds final values; rebuild the product part together with D */
            for (int i = nb; i < nm; i++) mom[i] = 0;
            for (int t = 0; t < nt; t++) {
                const int *row = times + 4 * t;
                T v0 = mom[row[0]], v1 = mom[row[1]], mu_ = (T)row[2];
                mom[row[3]] += mu_ * v0 * v1;
                D[row[3]] += D[row[0]] * mu_ * v1 + D[row[1]] * mu_ * v0;
            }
            NAME(mtp_adjoint)(&m, mom, lin, qs, adj);
            for (int t = 0; t < nt; t++) {
                const int *row = times + 4 * t;
                G[row[1]] += (T)row[2] * adj[row[3]] * D[row[0]];
                G[row[0]] += (T)row[2] * adj[row[3]] * D[row[1]];
            }
            for (int t = nt - 1; t >= 0; t--) {
                const int *row = times + 4 * t;
                G[row[0]] += G[row[3]] * (T)row[2] * mom[row[1]];
                G[row[1]] += G[row[3]] * (T)row[2] * mom[row[0]];
            }
            for (int j = 0; j < nn; j++) {
                const T *v = rc + 3 * j;
                T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
                if (r > rmax) continue;
                int nj = fn[j], tj = types[nj];
                T rinv = 1 / r, p[3];
                for (int a = 0; a < 3; a++) {
                    p[a] = cf * (fm[3 * ci + a] - fd[3 * ci + a]) - cf * (fm[3 * nj + a] - fd[3 * nj + a]);
                    for (int c = 0; c < 3; c++) p[a] -= cv * dV[3 * a + c] * v[c];
                }
                NAME(mtp_radial)(r, rmax, rmin, cs, q, dq);
                dist_pw[0] = 1; pw[0][0] = pw[1][0] = pw[2][0] = 1;
                for (int k = 1; k <= kmax; k++) { dist_pw[k] = dist_pw[k - 1] * r; for (int c = 0; c < 3; c++) pw[c][k] = pw[c][k - 1] * v[c]; }
                for (int i = 0; i < nb; i++) {
                    const int *al = basic + 4 * i;
                    int mu = al[0], k = al[1] + al[2] + al[3];
                    T C = 1 / dist_pw[k], Bm = pw[0][al[1]] * pw[1][al[2]] * pw[2][al[3]];
                    T Bd[3] = {0, 0, 0};
                    if (al[1]) Bd[0] = al[1] * pw[0][al[1] - 1] * pw[1][al[2]] * pw[2][al[3]];
                    if (al[2]) Bd[1] = al[2] * pw[0][al[1]] * pw[1][al[2] - 1] * pw[2][al[3]];
                    if (al[3]) Bd[2] = al[3] * pw[0][al[1]] * pw[1][al[2]] * pw[2][al[3] - 1];
                    T *go = gco + ((size_t)(ti * ntypes + tj) * nmus + mu) * cs;
                    for (int xi = 0; xi < cs; xi++) {
                        T A = q[xi] * scaling, Ad = dq[xi] * scaling;
                        T acc = (ce * adj[i] + G[i]) * A * Bm * C;
                        for (int a = 0; a < 3; a++) {
                            T Cd = -k * C * rinv * rinv * v[a];
                            acc += p[a] * adj[i] * (Ad * v[a] * rinv * Bm * C + A * Bd[a] * C + A * Bm * Cd);
                        }
                        go[xi] += acc;
                    }
                }
            }
            for (int s = 0; s < ns; s++) gli[s] += (ce * mom[map[s]] + D[map[s]]) / qs[s];
            gbi[ti] += ce;
        }
    }
    free(mom); free(adj); free(D); free(G); free(mder);
    return 0;
}
int NAME2(orc_mtp_ef_loss_backward)(T *dco, T *dli, T *dbi, T ew, T fw, const T *e_ml, const T *e_dft, const T *f_ml,
                                    const T *f_dft, int cs, T scaling, const T *coeffs, const T *lin, const T *bias,
                                    TAB_DECL, NB_DECL, T rmax, T rmin, const T *qs)
{
    return NAME2(orc_mtp_loss_backward)(dco, dli, dbi, ew, fw, 0, e_ml, e_dft, f_ml, f_dft, NULL, NULL, cs, scaling, coeffs, lin, bias,
                                        nm, nb, basic, nt, times, ns, map, nmus, B, npad, binum, bilist, bnumneigh, bfirstneigh, brcs,
                                        btypes, ntypes, type_map, umax, nghost, rmax, rmin, qs);
}

/* ---------------------------------------------------------------------------------------
 * NEP (3-body). Radial functions descriptor/nep/include/basis.h:137-159 (cosine switch),
 * :300-333 (f_k = (T_k(x)+1)/2, x = 2(r/rc-1)^2-1), :519-530; harmonics as homogeneous
 * polynomials nep_utilities.h:100-383; sums nepBasis.h:57-196; network and forces
 * nep.h:320-529.
 * ------------------------------------------------------------------------------------- */
static void NAME(nep_radial)(T r, T rc, int cs, T *f, T *df)
{
    T fc = 0, dfc = 0;
    if (r <= rc) { fc = (T)(0.5 * (1 + cos(M_PI * r / rc))); dfc = (T)(-0.5 * sin(M_PI * r / rc) * M_PI / rc); }
    T x = 2 * (r / rc - 1) * (r / rc - 1) - 1, xc = (T)4.0 / rc * (r / rc - 1);
    T t0 = 1, t1 = x, d0 = 0, d1 = 1;
    for (int k = 0; k < cs; k++) {
        T t, d;
        if (k == 0) { t = 1; d = 0; }
        else if (k == 1) { t = x; d = 1; }
        else { t = 2 * x * t1 - t0; d = 2 * t1 + 2 * x * d1 - d0; t0 = t1; t1 = t; d0 = d1; d1 = d; }
        T v = (t + 1) * (T)0.5, dv = xc * (d * (T)0.5);
        f[k] = fc * v;
        df[k] = dfc * v + fc * dv;
    }
}

/* 24 harmonic polynomials b[l*l-1+m'] (l=1..4) and their Cartesian gradients, written from
 * the closed forms in terms of x, y, z and r2 = x^2+y^2+z^2; the gradients are the full
 * Cartesian gradients (r2 differentiated too), as tabulated in nep_utilities.h:206-383. */
static void NAME(nep_blm)(const T *v, T r, T *b, T (*g)[3])
{
    T x = v[0], y = v[1], z = v[2], r2 = r * r, x2 = x * x, y2 = y * y, z2 = z * z;
    int k = 0;
#define SET(val, gx, gy, gz) do { b[k] = (val); g[k][0] = (gx); g[k][1] = (gy); g[k][2] = (gz); k++; } while (0)
    /* l = 1 */
    SET(z, 0, 0, 1); SET(x, 1, 0, 0); SET(y, 0, 1, 0);
    /* l = 2 */
    SET(3 * z2 - r2, -2 * x, -2 * y, 4 * z);
    SET(x * z, z, 0, x);
    SET(y * z, 0, z, y);
    SET(x2 - y2, 2 * x, -2 * y, 0);
    SET(2 * x * y, 2 * y, 2 * x, 0);
    /* l = 3 */
    SET((5 * z2 - 3 * r2) * z, -6 * x * z, -6 * y * z, 9 * z2 - 3 * r2);
    SET((5 * z2 - r2) * x, -2 * x2 + 5 * z2 - r2, -2 * x * y, 8 * x * z);
    SET((5 * z2 - r2) * y, -2 * x * y, -2 * y2 + 5 * z2 - r2, 8 * y * z);
    SET((x2 - y2) * z, 2 * x * z, -2 * y * z, x2 - y2);
    SET(2 * x * y * z, 2 * y * z, 2 * x * z, 2 * x * y);
    SET((x2 - 3 * y2) * x, 3 * x2 - 3 * y2, -6 * x * y, 0);
    SET((3 * x2 - y2) * y, 6 * x * y, 3 * x2 - 3 * y2, 0);
    /* l = 4 */
    SET((35 * z2 - 30 * r2) * z2 + 3 * r2 * r2, -60 * x * z2 + 12 * r2 * x, -60 * y * z2 + 12 * r2 * y, 80 * z2 * z - 48 * r2 * z);
    SET((7 * z2 - 3 * r2) * x * z, -6 * x2 * z + 7 * z2 * z - 3 * r2 * z, -6 * x * y * z, 15 * x * z2 - 3 * r2 * x);
    SET((7 * z2 - 3 * r2) * y * z, -6 * x * y * z, -6 * y2 * z + 7 * z2 * z - 3 * r2 * z, 15 * y * z2 - 3 * r2 * y);
    SET((7 * z2 - r2) * (x2 - y2), -2 * x2 * x + 2 * x * y2 + 14 * x * z2 - 2 * r2 * x, -2 * x2 * y + 2 * y2 * y - 14 * y * z2 + 2 * r2 * y, 12 * z * (x2 - y2));
    SET((7 * z2 - r2) * 2 * x * y, -4 * x2 * y + 14 * y * z2 - 2 * r2 * y, -4 * x * y2 + 14 * x * z2 - 2 * r2 * x, 24 * x * y * z);
    SET((x2 - 3 * y2) * x * z, 3 * x2 * z - 3 * y2 * z, -6 * x * y * z, (x2 - 3 * y2) * x);
    SET((3 * x2 - y2) * y * z, 6 * x * y * z, 3 * x2 * z - 3 * y2 * z, (3 * x2 - y2) * y);
    SET((x2 - y2) * (x2 - y2) - 4 * x2 * y2, 4 * x2 * x - 12 * x * y2, 4 * y2 * y - 12 * x2 * y, 0);
    SET(4 * (x2 - y2) * x * y, 12 * x2 * y - 4 * y2 * y, 4 * x2 * x - 12 * x * y2, 0);
#undef SET
}

/* 3-body coefficients, nep_utilities.h:25-31: entries with an `f` suffix there are float
 * literals widened to double; reproduced with the same rounding. */
static const double NAME(C3B)[24] = {
    0.238732414637843, (double)0.119366207318922f, (double)0.119366207318922f, (double)0.099471839432435f,
    0.596831036594608, (double)0.596831036594608f, (double)0.149207759148652f, (double)0.149207759148652f,
    0.139260575205408, (double)0.104445431404056f, (double)0.104445431404056f, (double)1.044454314040563f,
    1.044454314040563, (double)0.174075719006761f, (double)0.174075719006761f, (double)0.011190581936149f,
    0.223811638722978, (double)0.223811638722978f, (double)0.111905819361489f, (double)0.111905819361489f,
    1.566681471060845, (double)1.566681471060845f, (double)0.195835183882606f, (double)0.195835183882606f};

typedef struct { int cs, nr, na, lmax, ntypes; T rcr, rca; const T *coeffs; } NAME(nepdef);

/* descriptors q[nr + na*lmax], sums S[na*nlm]; optional per-pair gradients dq[nr][nn][3], dS[na*nlm][nn][3] */
static void NAME(nep_desc)(const NAME(nepdef) *m, int ti, int nn, const int *fn, const T *rc, const int *types,
                           T *q, T *S, T *dq, T *dS)
{
    int nlm = m->lmax * m->lmax + 2 * m->lmax, nd = m->nr + m->na * m->lmax;
    T fr[64], dfr[64], fa[64], dfa[64], b[24], gb[24][3];
    memset(q, 0, sizeof(T) * nd); memset(S, 0, sizeof(T) * m->na * nlm);
    if (dq) memset(dq, 0, sizeof(T) * 3 * (size_t)m->nr * nn);
    if (dS) memset(dS, 0, sizeof(T) * 3 * (size_t)m->na * nlm * nn);
    for (int j = 0; j < nn; j++) {
        const T *v = rc + 3 * j;
        T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
        if (r > m->rcr) continue;
        int tj = types[fn[j]];
        T rinv = 1 / r;
        NAME(nep_radial)(r, m->rcr, m->cs, fr, dfr);
        NAME(nep_radial)(r, m->rca, m->cs, fa, dfa);
        const T *co = m->coeffs + (size_t)(ti * m->ntypes + tj) * (m->nr + m->na) * m->cs;
        for (int n = 0; n < m->nr; n++)
            for (int xi = 0; xi < m->cs; xi++) {
                q[n] += co[n * m->cs + xi] * fr[xi];
                if (dq) for (int a = 0; a < 3; a++) dq[((size_t)n * nn + j) * 3 + a] += co[n * m->cs + xi] * dfr[xi] * v[a] * rinv;
            }
        if (r <= m->rca && m->lmax > 0) {
            NAME(nep_blm)(v, r, b, gb);
            T rp[5] = {1, r, r * r, r * r * r, r * r * r * r};
            for (int mu = 0; mu < m->na; mu++)
                for (int l = 1; l <= m->lmax; l++) {
                    T C = 1 / rp[l], pre = -l / (rp[l] * r) * rinv;
                    for (int mp = 0; mp < 2 * l + 1; mp++) {
                        int lm = l * l - 1 + mp, si = mu * nlm + lm;
                        for (int xi = 0; xi < m->cs; xi++) {
                            T c = co[(m->nr + mu) * m->cs + xi];
                            S[si] += c * fa[xi] * b[lm] * C;
                            if (dS) for (int a = 0; a < 3; a++)
                                dS[((size_t)si * nn + j) * 3 + a] += c * (dfa[xi] * v[a] * rinv * b[lm] * C + fa[xi] * gb[lm][a] * C + fa[xi] * b[lm] * pre * v[a]);
                        }
                    }
                }
        }
    }
    for (int mu = 0; mu < m->na; mu++)
        for (int l = 1; l <= m->lmax; l++)
            for (int mp = 0; mp < 2 * l + 1; mp++) {
                int lm = l * l - 1 + mp;
                T s = S[mu * nlm + lm];
                q[m->nr + mu * m->lmax + l - 1] += (mp == 0 ? 1 : 2) * (T)NAME(C3B)[lm] * s * s;
            }
}

static void NAME(nep_efv_impl)(T *betot, T *bforce, T *bvirial, int cs, int nr, int na, int lmax, int nneu, const T *coeffs,
                               const T *w0, const T *b0, const T *w1, const T *bias, NB_DECL, T rcr, T rca, const T *qs)
{
    (void)type_map;
    NAME(nepdef) m = {cs, nr, na, lmax, ntypes, rcr, rca, coeffs};
    int nlm = lmax * lmax + 2 * lmax, nd = nr + na * lmax, nS = na * nlm;
    T *q = (T *)malloc(sizeof(T) * nd), *S = (T *)malloc(sizeof(T) * (nS + 1)), *dEq = (T *)malloc(sizeof(T) * nd), *dES = (T *)malloc(sizeof(T) * (nS + 1));
    T *dq = (T *)malloc(sizeof(T) * 3 * (size_t)nr * umax + 8), *dS = (T *)malloc(sizeof(T) * 3 * (size_t)nS * umax + 8);
    for (int b = 0; b < B; b++) {
        T *force = bforce + (size_t)b * (npad + nghost) * 3;
        const int *types = btypes + (size_t)b * (npad + nghost);
        T etot = 0, vir[9] = {0};
        for (int ii = 0; ii < binum[b]; ii++) {
            size_t slot = (size_t)b * npad + ii;
            int ci = bilist[slot], nn = bnumneigh[slot], ti = types[ci];
            const int *fn = bfirstneigh + slot * umax;
            const T *rc = brcs + slot * umax * 3;
            NAME(nep_desc)(&m, ti, nn, fn, rc, types, q, S, dq, dS);
            const T *W0 = w0 + (size_t)ti * nneu * nd, *B0 = b0 + (size_t)ti * nneu, *W1 = w1 + (size_t)ti * nneu;
            T es = bias[ti];
            memset(dEq, 0, sizeof(T) * nd);
            for (int p = 0; p < nneu; p++) {
                T h = 0;
                for (int k = 0; k < nd; k++) h += W0[p * nd + k] * q[k] / qs[k];
                h += B0[p];
                T th = (T)tanh((double)h);
                es += W1[p] * th;
                for (int k = 0; k < nd; k++) dEq[k] += W1[p] * (1 - th * th) * W0[p * nd + k] / qs[k];
            }
            etot += es;
            for (int mu = 0; mu < na; mu++)
                for (int l = 1; l <= lmax; l++)
                    for (int mp = 0; mp < 2 * l + 1; mp++) {
                        int lm = l * l - 1 + mp;
                        dES[mu * nlm + lm] = (mp == 0 ? 1 : 2) * dEq[nr + mu * lmax + l - 1] * 2 * (T)NAME(C3B)[lm] * S[mu * nlm + lm];
                    }
            for (int j = 0; j < nn; j++) {
                const T *v = rc + 3 * j;
                T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
                if (r > rcr) continue;
                for (int a = 0; a < 3; a++) {
                    T g = 0;
                    for (int k = 0; k < nr; k++) g += dEq[k] * dq[((size_t)k * nn + j) * 3 + a];
                    for (int s = 0; s < nS; s++) g += dES[s] * dS[((size_t)s * nn + j) * 3 + a];
                    force[3 * ci + a] += g;
                    force[3 * fn[j] + a] -= g;
                    for (int c = 0; c < 3; c++) vir[3 * a + c] -= g * v[c];
                }
            }
        }
        betot[b] += etot;
        if (bvirial) for (int k = 0; k < 9; k++) bvirial[9 * b + k] += vir[k];
    }
    free(q); free(S); free(dEq); free(dES); free(dq); free(dS);
}
int NAME2(orc_nep_efv)(T *betot, T *bforce, T *bvirial, int cs, int nr, int na, int lmax, int nneu, const T *coeffs, const T *w0,
                       const T *b0, const T *w1, const T *bias, NB_DECL, T rcr, T rca, const T *qs)
{
    NAME(nep_efv_impl)(betot, bforce, bvirial, cs, nr, na, lmax, nneu, coeffs, w0, b0, w1, bias, B, npad, binum, bilist, bnumneigh,
                       bfirstneigh, brcs, btypes, ntypes, type_map, umax, nghost, rcr, rca, qs);
    return 0;
}
int NAME2(orc_nep_ef)(T *betot, T *bforce, int cs, int nr, int na, int lmax, int nneu, const T *coeffs, const T *w0, const T *b0,
                      const T *w1, const T *bias, NB_DECL, T rcr, T rca, const T *qs)
{
    NAME(nep_efv_impl)(betot, bforce, NULL, cs, nr, na, lmax, nneu, coeffs, w0, b0, w1, bias, B, npad, binum, bilist, bnumneigh,
                       bfirstneigh, brcs, btypes, ntypes, type_map, umax, nghost, rcr, rca, qs);
    return 0;
}
int NAME2(orc_nep_descriptors)(T *bdesc, int cs, int nr, int na, int lmax, const T *coeffs, NB_DECL, T rcr, T rca)
{
    (void)type_map; (void)nghost;
    NAME(nepdef) m = {cs, nr, na, lmax, ntypes, rcr, rca, coeffs};
    int nlm = lmax * lmax + 2 * lmax, nd = nr + na * lmax;
    T *q = (T *)malloc(sizeof(T) * nd), *S = (T *)malloc(sizeof(T) * (na * nlm + 1));
    for (int b = 0; b < B; b++) {
        const int *types = btypes + (size_t)b * npad;
        for (int ii = 0; ii < binum[b]; ii++) {
            size_t slot = (size_t)b * npad + ii;
            NAME(nep_desc)(&m, types[bilist[slot]], bnumneigh[slot], bfirstneigh + slot * umax, brcs + slot * umax * 3, types, q, S, NULL, NULL);
            memcpy(bdesc + slot * nd, q, sizeof(T) * nd);
        }
    }
    free(q); free(S);
    return 0;
}

/* NEP loss gradient w.r.t. coeffs, w0, b0, w1, type_bias, per structure (descriptor/nep/include/nepLoss.h:
 * find_loss_backward / find_ef_loss_backward; launcher nepLoss_cpu_launcher.h:213-330). Derivation used here:
 * with lam = 2 e_w/n (E - E*), P_a = 2 f_w/(3n) (F_a - F*_a), Qm = 2 v_w/(9n) (V - V*), the force and virial
 * terms of the loss are  Phi = sum_ij g_ij . p_ij  with  p_ij = P_i - P_j - Qm r_ij  and g_ij the pair gradient,
 * so  dL/dtheta = lam dE/dtheta + dPhi/dtheta  and, per atom,  Phi_i = sum_k (dE_i/dq_k) u_k  with
 * u_k = sum_j dq_k/dr_ij . p_ij  (directional derivative of the descriptors along p). */
int NAME2(orc_nep_loss_backward)(T *dco, T *dw0, T *db0, T *dw1, T *dbi, T ew, T fw, T vw, const T *e_ml, const T *e_dft,
                                 const T *f_ml, const T *f_dft, const T *v_ml, const T *v_dft, int cs, int nr, int na, int lmax,
                                 int nneu, const T *coeffs, const T *w0, const T *b0, const T *w1, const T *bias, NB_DECL, T rcr, T rca, const T *qs)
{
    (void)type_map; (void)nghost; (void)bias;
    NAME(nepdef) m = {cs, nr, na, lmax, ntypes, rcr, rca, coeffs};
    const int nlm = lmax * lmax + 2 * lmax, nd = nr + na * lmax, nS = na * nlm, nfun = nr + na;
    const int ncoef = ntypes * ntypes * nfun * cs;
    T *q = (T *)malloc(sizeof(T) * nd), *S = (T *)malloc(sizeof(T) * (nS + 1)), *u = (T *)malloc(sizeof(T) * nd), *DS = (T *)malloc(sizeof(T) * (nS + 1));
    T *a = (T *)malloc(sizeof(T) * nd), *be = (T *)malloc(sizeof(T) * nd), *th = (T *)malloc(sizeof(T) * nneu), *sp = (T *)malloc(sizeof(T) * nneu);
    T *dq = (T *)malloc(sizeof(T) * 3 * (size_t)nr * umax + 8), *dS = (T *)malloc(sizeof(T) * 3 * (size_t)nS * umax + 8);
    T *p = (T *)malloc(sizeof(T) * 3 * (size_t)umax + 8);
    T fr[64], dfr[64], fa[64], dfa[64], bl[24], gb[24][3];
    memset(dco, 0, sizeof(T) * (size_t)B * ncoef); memset(dw0, 0, sizeof(T) * (size_t)B * ntypes * nneu * nd);
    memset(db0, 0, sizeof(T) * (size_t)B * ntypes * nneu); memset(dw1, 0, sizeof(T) * (size_t)B * ntypes * nneu);
    memset(dbi, 0, sizeof(T) * (size_t)B * ntypes);
    for (int b = 0; b < B; b++) {
        const int n = binum[b];
        const int *types = btypes + (size_t)b * npad;
        const T *fm = f_ml + (size_t)b * npad * 3, *fd = f_dft + (size_t)b * npad * 3;
        const T lam = 2 * ew / n * (e_ml[b] - e_dft[b]), cf = 2 * fw / (3 * n), cv = v_ml ? 2 * vw / (9 * n) : 0;
        T dV[9] = {0};
        if (v_ml) for (int k = 0; k < 9; k++) dV[k] = v_ml[9 * b + k] - v_dft[9 * b + k];
        T *gco = dco + (size_t)b * ncoef;
        for (int ii = 0; ii < n; ii++) {
            const size_t slot = (size_t)b * npad + ii;
            const int ci = bilist[slot], nn = bnumneigh[slot], ti = types[ci];
            const int *fn = bfirstneigh + slot * umax;
            const T *rc = brcs + slot * umax * 3;
            NAME(nep_desc)(&m, ti, nn, fn, rc, types, q, S, dq, dS);
            for (int j = 0; j < nn; j++)
                for (int c = 0; c < 3; c++) {
                    T v = cf * (fm[3 * ci + c] - fd[3 * ci + c]) - cf * (fm[3 * fn[j] + c] - fd[3 * fn[j] + c]);
                    for (int d = 0; d < 3; d++) v -= cv * dV[3 * c + d] * rc[3 * j + d];
                    p[3 * j + c] = v;
                }
            /* directional derivatives of the sums and of the descriptors */
            memset(u, 0, sizeof(T) * nd); memset(DS, 0, sizeof(T) * (nS + 1));
            for (int j = 0; j < nn; j++) {
                const T *v = rc + 3 * j;
                T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
                if (r > rcr) continue;
                for (int c = 0; c < 3; c++) {
                    for (int k = 0; k < nr; k++) u[k] += dq[((size_t)k * nn + j) * 3 + c] * p[3 * j + c];
                    for (int s2 = 0; s2 < nS; s2++) DS[s2] += dS[((size_t)s2 * nn + j) * 3 + c] * p[3 * j + c];
                }
            }
            for (int mu = 0; mu < na; mu++)
                for (int l = 1; l <= lmax; l++)
                    for (int mp = 0; mp < 2 * l + 1; mp++) {
                        int lm = l * l - 1 + mp;
                        u[nr + mu * lmax + l - 1] += (mp == 0 ? 1 : 2) * 2 * (T)NAME(C3B)[lm] * S[mu * nlm + lm] * DS[mu * nlm + lm];
                    }
            /* network: a = dE/dq, s_p = (W0 u~)_p, beta_k = dPhi/dq~_k */
            const T *W0 = w0 + (size_t)ti * nneu * nd, *B0 = b0 + (size_t)ti * nneu, *W1 = w1 + (size_t)ti * nneu;
            T *gw0 = dw0 + ((size_t)b * ntypes + ti) * nneu * nd, *gb0 = db0 + ((size_t)b * ntypes + ti) * nneu, *gw1 = dw1 + ((size_t)b * ntypes + ti) * nneu;
            memset(a, 0, sizeof(T) * nd); memset(be, 0, sizeof(T) * nd);
            for (int pn = 0; pn < nneu; pn++) {
                T h = 0, sv = 0;
                for (int k = 0; k < nd; k++) { h += W0[pn * nd + k] * q[k] / qs[k]; sv += W0[pn * nd + k] * u[k] / qs[k]; }
                h += B0[pn];
                th[pn] = (T)tanh((double)h); sp[pn] = sv;
                const T d1 = 1 - th[pn] * th[pn], d2 = -2 * th[pn] * d1;
                for (int k = 0; k < nd; k++) { a[k] += W1[pn] * d1 * W0[pn * nd + k] / qs[k]; be[k] += W1[pn] * sv * d2 * W0[pn * nd + k] / qs[k]; }
                gw1[pn] += lam * th[pn] + d1 * sv;
                gb0[pn] += lam * W1[pn] * d1 + W1[pn] * sv * d2;
                for (int k = 0; k < nd; k++)
                    gw0[pn * nd + k] += (lam * W1[pn] * d1 + W1[pn] * sv * d2) * q[k] / qs[k] + W1[pn] * d1 * u[k] / qs[k];
            }
            dbi[(size_t)b * ntypes + ti] += lam;
            /* coefficients: dL/dc = sum_k (lam a_k + beta_k) dq_k/dc + a_k du_k/dc */
            for (int j = 0; j < nn; j++) {
                const T *v = rc + 3 * j;
                T r = (T)sqrt((double)(v[0] * v[0] + v[1] * v[1] + v[2] * v[2]));
                if (r > rcr) continue;
                const int tj = types[fn[j]];
                const T rinv = 1 / r, vp = (v[0] * p[3 * j] + v[1] * p[3 * j + 1] + v[2] * p[3 * j + 2]) * rinv;
                NAME(nep_radial)(r, rcr, cs, fr, dfr);
                NAME(nep_radial)(r, rca, cs, fa, dfa);
                T *go = gco + (size_t)(ti * ntypes + tj) * nfun * cs;
                for (int k = 0; k < nr; k++)
                    for (int xi = 0; xi < cs; xi++) go[k * cs + xi] += (lam * a[k] + be[k]) * fr[xi] + a[k] * dfr[xi] * vp;
                if (r <= rca && lmax > 0) {
                    NAME(nep_blm)(v, r, bl, gb);
                    T rp[5] = {1, r, r * r, r * r * r, r * r * r * r};
                    for (int mu = 0; mu < na; mu++)
                        for (int l = 1; l <= lmax; l++) {
                            const int k = nr + mu * lmax + l - 1;
                            const T C = 1 / rp[l], pre = -l / (rp[l] * r) * rinv;
                            for (int mp = 0; mp < 2 * l + 1; mp++) {
                                const int lm = l * l - 1 + mp, si = mu * nlm + lm;
                                const T w2c = (mp == 0 ? 1 : 2) * 2 * (T)NAME(C3B)[lm];
                                const T gp = gb[lm][0] * p[3 * j] + gb[lm][1] * p[3 * j + 1] + gb[lm][2] * p[3 * j + 2];
                                for (int xi = 0; xi < cs; xi++) {
                                    const T dSc = fa[xi] * bl[lm] * C;                                   /* dS/dc  */
                                    const T dDSc = dfa[xi] * vp * bl[lm] * C + fa[xi] * gp * C + fa[xi] * bl[lm] * pre * vp * r;   /* dDS/dc */
                                    go[(nr + mu) * cs + xi] += (lam * a[k] + be[k]) * w2c * S[si] * dSc + a[k] * w2c * (dSc * DS[si] + S[si] * dDSc);
                                }
                            }
                        }
                }
            }
        }
    }
    free(q); free(S); free(u); free(DS); free(a); free(be); free(th); free(sp); free(dq); free(dS); free(p);
    return 0;
}
int NAME2(orc_nep_ef_loss_backward)(T *dco, T *dw0, T *db0, T *dw1, T *dbi, T ew, T fw, const T *e_ml, const T *e_dft, const T *f_ml,
                                    const T *f_dft, int cs, int nr, int na, int lmax, int nneu, const T *coeffs, const T *w0,
                                    const T *b0, const T *w1, const T *bias, NB_DECL, T rcr, T rca, const T *qs)
{
    return NAME2(orc_nep_loss_backward)(dco, dw0, db0, dw1, dbi, ew, fw, 0, e_ml, e_dft, f_ml, f_dft, NULL, NULL, cs, nr, na, lmax, nneu,
                                        coeffs, w0, b0, w1, bias, B, npad, binum, bilist, bnumneigh, bfirstneigh, brcs, btypes, ntypes,
                                        type_map, umax, nghost, rcr, rca, qs);
}

/* fvt values: fvt/include/force_sr.h:50-81, virial_sr.h:24-51 */
int NAME2(orc_fvt_force)(T *force, int inum, const int *ilist, const int *numneigh, const int *firstneigh, int nghost, int umax, const T *de)
{
    memset(force, 0, sizeof(T) * 3 * (size_t)(inum + nghost));
    for (int ii = 0; ii < inum; ii++)
        for (int j = 0; j < numneigh[ii]; j++)
            for (int a = 0; a < 3; a++) {
                T g = de[((size_t)ii * umax + j) * 3 + a];
                force[3 * ilist[ii] + a] += g;
                force[3 * firstneigh[(size_t)ii * umax + j] + a] -= g;
            }
    return 0;
}
int NAME2(orc_fvt_virial)(T *virial, int inum, const int *numneigh, const T *rcs, int umax, const T *de)
{
    memset(virial, 0, sizeof(T) * 9);
    for (int ii = 0; ii < inum; ii++)
        for (int j = 0; j < numneigh[ii]; j++)
            for (int a = 0; a < 3; a++)
                for (int c = 0; c < 3; c++)
                    virial[3 * a + c] -= de[((size_t)ii * umax + j) * 3 + a] * rcs[((size_t)ii * umax + j) * 3 + c];
    return 0;
}

/* ZBL pair correction, complete form (energy, force on the centre atom, virial; accumulates into the
 * outputs): pair functions of descriptor/correction/include/zbl.h:276-395 applied per directed pair as
 * in descriptor/correction/gpu/include/zbl.cuh:423-500. Expressions that involve the double constant
 * K_C_SP or std::pow(T, int) are evaluated in double, as in the reference. */
int NAME2(orc_zbl_efv)(T *etot, T *force, T *virial, int inum, const int *ilist, const int *numneigh, const int *firstneigh,
                       const T *rcs, const int *types, int ntypes, const int *type_map, int umax, int nghost, T rmax, T rmin,
                       const T *cks, const T *dks)
{
    const double KC = 14.399645;
    (void)nghost;
    for (int ii = 0; ii < inum; ii++) {
        const int ci = ilist[ii], ti = types[ci];
        for (int jj = 0; jj < numneigh[ii]; jj++) {
            const T *v = rcs + ((size_t)ii * umax + jj) * 3;
            const int tj = types[firstneigh[(size_t)ii * umax + jj]];
            const T dist = (T)sqrt((double)v[0] * v[0] + (double)v[1] * v[1] + (double)v[2] * v[2]);
            if (dist > rmax) continue;
            const int Zi = type_map[ti], Zj = type_map[tj];
            const T *ck = cks + 4 * (ti * ntypes + tj), *dk = dks + 4 * (ti * ntypes + tj);
            const T a = (T)(0.46848 / (pow((double)Zi, 0.23) + pow((double)Zj, 0.23)));
            const T x = dist / a;
            T phi = 0, dphi = 0;
            for (int k = 0; k < 4; k++) {
                phi += ck[k] * (T)exp((double)(-dk[k] * x));
                dphi += -ck[k] * dk[k] / a * (T)exp((double)(-dk[k] * dist / a));
            }
            T sw, dsw;
            if (dist < rmin) { sw = 1; dsw = 0; }
            else {
                const T uu = (dist - rmin) / (rmax - rmin);
                sw = (T)((double)uu * uu * uu * (-6 * (double)uu * uu + 15 * uu - 10) + 1);
                dsw = (T)(1 / (rmax - rmin) * (-30 * (double)uu * uu * uu * uu + 60 * (double)uu * uu * uu - 30 * (double)uu * uu));
            }
            const T A = (T)(KC * Zi * Zj / dist), dA = (T)(-KC * Zi * Zj / ((double)dist * dist));
            *etot += (T)(0.5 * (T)(KC * (Zi * Zj) / dist * phi * sw));
            const T dE = dA * phi * sw + A * dphi * sw + A * phi * dsw;
            for (int c = 0; c < 3; c++) force[3 * ci + c] += dE * v[c] / dist;
            if (virial)
                for (int c = 0; c < 3; c++)
                    for (int d = 0; d < 3; d++) virial[3 * c + d] += (T)(-0.5 * v[c] * (dE * v[d] / dist));
        }
    }
    return 0;
}

/* dataset statistics: descriptor/fitutils/include/descriptorsStatistics.h:76-205, targetStatistics.h:44-80
 * (same two-pass definition; sums in double) */
int NAME2(orc_desc_stats_each)(int *natoms, T *mean, T *m2, int B, int npad, int nd, const int *binum, const int *bilist,
                               const int *btypes, int ntypes, const T *bdesc)
{
    for (int t = 0; t < ntypes; t++) {
        for (int k = 0; k < nd; k++) {
            double s = 0, c = 0, q = 0;
            for (int b = 0; b < B; b++)
                for (int ii = 0; ii < binum[b]; ii++)
                    if (!btypes || btypes[(size_t)b * npad + bilist[(size_t)b * npad + ii]] == t) { s += bdesc[((size_t)b * npad + ii) * nd + k]; c += 1; }
            T mu = c > 0 ? (T)(s / c) : 0;
            for (int b = 0; b < B; b++)
                for (int ii = 0; ii < binum[b]; ii++)
                    if (!btypes || btypes[(size_t)b * npad + bilist[(size_t)b * npad + ii]] == t) {
                        double d = (double)(T)(bdesc[((size_t)b * npad + ii) * nd + k] - mu);
                        q += d * d;
                    }
            mean[(size_t)t * nd + k] = mu; m2[(size_t)t * nd + k] = (T)q;
            if (k == 0) natoms[t] = (int)c;
        }
    }
    return 0;
}
int NAME2(orc_desc_stats_all)(int *natoms, T *mean, T *m2, int B, int npad, int nd, const int *binum, const T *bdesc)
{
    return NAME2(orc_desc_stats_each)(natoms, mean, m2, B, npad, nd, binum, NULL, NULL, 1, bdesc);
}
int NAME2(orc_desc_maxmin)(T *mx, T *mn, int B, int npad, int nd, const int *binum, const T *bdesc)
{
    for (int k = 0; k < nd; k++) {
        T a = (T)1.17549435e-38f, z = (T)3.40282347e+38f;   /* FLT_MIN, FLT_MAX: the reference's starting values */
        for (int b = 0; b < B; b++)
            for (int ii = 0; ii < binum[b]; ii++) {
                T x = bdesc[((size_t)b * npad + ii) * nd + k];
                a = a > x ? a : x; z = z < x ? z : x;
            }
        mx[k] = a; mn[k] = z;
    }
    return 0;
}
int NAME2(orc_target_stats)(int *natoms, T *out3, int B, int npad, const int *binum, const T *etot, const T *force)
{
    double n = 0, es = 0, f2 = 0, q = 0;
    for (int b = 0; b < B; b++) {
        n += binum[b]; es += (double)(T)(etot[b] / binum[b]);
        for (int ii = 0; ii < binum[b]; ii++)
            for (int a = 0; a < 3; a++) { double f = force[((size_t)b * npad + ii) * 3 + a]; f2 += f * f; }
    }
    T mu = (T)(es / B);
    for (int b = 0; b < B; b++) { double d = (double)(T)(etot[b] / binum[b] - mu); q += d * d; }
    natoms[0] = (int)n; out3[0] = mu; out3[1] = (T)q; out3[2] = (T)f2;
    return 0;
}

#undef NB_DECL
#undef TAB_DECL
