// Host side of the linear-MTP path: error state, .almtp parser, alpha-table compiler.
#include "mtp_program.cuh"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

namespace ai2b {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count()
{
    static std::mutex mu;
    static int counts[MAX_DEVICES] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    const bool cached = dev >= 0 && dev < MAX_DEVICES;
    std::lock_guard<std::mutex> guard(mu);
    if (cached && counts[dev] > 0) return counts[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (cached) counts[dev] = n;
    return n;
}

}  // namespace ai2b

using namespace ai2b;

extern "C" const char *ai2b_last_error_string(void) { return ai2b::g_err; }
extern "C" int ai2b_version(void) { return 100; }

// ---------------------------------------------------------------------------------------------
// .almtp parser. Same fields, in the same order, as source/descriptor/mtpr/src/mtpParam.cc:80-200
// reads them; located here by key name rather than by skipping a fixed number of header lines.
// ---------------------------------------------------------------------------------------------
static bool find_key(const std::string &txt, const char *key, size_t &pos)
{
    size_t p = 0;
    const size_t klen = strlen(key);
    while ((p = txt.find(key, p)) != std::string::npos) {
        bool word_start = (p == 0) || !(isalnum((unsigned char)txt[p - 1]) || txt[p - 1] == '_');
        size_t q = p + klen;
        while (q < txt.size() && (txt[q] == ' ' || txt[q] == '\t')) ++q;
        if (word_start && q < txt.size() && txt[q] == '=') {
            pos = q + 1;
            return true;
        }
        p += klen;
    }
    return false;
}

static bool read_int(const std::string &txt, const char *key, int &v)
{
    size_t pos;
    if (!find_key(txt, key, pos)) return false;
    v = (int)strtol(txt.c_str() + pos, nullptr, 10);
    return true;
}

static bool read_list(const std::string &txt, const char *key, std::vector<int> &out)
{
    size_t pos;
    if (!find_key(txt, key, pos)) return false;
    size_t end = txt.find('\n', pos);
    if (end == std::string::npos) end = txt.size();
    out.clear();
    const char *s = txt.c_str() + pos, *e = txt.c_str() + end;
    while (s < e) {
        if (isdigit((unsigned char)*s) || (*s == '-' && s + 1 < e && isdigit((unsigned char)s[1]))) {
            char *nx;
            out.push_back((int)strtol(s, &nx, 10));
            s = nx;
        } else {
            ++s;
        }
    }
    return true;
}

extern "C" int ai2b_mtp_parse_almtp(const char *filename, int *counts, int *basic, int *times, int *mapping)
{
    AI2B_REQUIRE(filename && counts, AI2B_ERR_INVALID, "ai2b_mtp_parse_almtp: NULL argument");
    std::ifstream in(filename);
    AI2B_REQUIRE(in.good(), AI2B_ERR_INVALID, "cannot open MTP template '%s'", filename);
    std::stringstream ss;
    ss << in.rdbuf();
    const std::string txt = ss.str();
    int nm, nb, nt, ns;
    std::vector<int> vb, vt, vm;
    bool ok = read_int(txt, "alpha_moments_count", nm) && read_int(txt, "alpha_index_basic_count", nb) &&
              read_list(txt, "alpha_index_basic", vb) && read_int(txt, "alpha_index_times_count", nt) &&
              read_list(txt, "alpha_index_times", vt) && read_int(txt, "alpha_scalar_moments", ns) &&
              read_list(txt, "alpha_moment_mapping", vm);
    AI2B_REQUIRE(ok, AI2B_ERR_INVALID, "'%s' is not an MTP template (missing alpha_* field)", filename);
    AI2B_REQUIRE((int)vb.size() == 4 * nb && (int)vt.size() == 4 * nt && (int)vm.size() == ns, AI2B_ERR_INVALID,
                 "'%s': table sizes do not match their counts", filename);
    int nmus = 0;
    for (int i = 0; i < nb; i++) nmus = std::max(nmus, vb[4 * i] + 1);   // mtpParam.cc:549-556
    counts[0] = nm; counts[1] = nb; counts[2] = nt; counts[3] = ns; counts[4] = nmus;
    if (basic) memcpy(basic, vb.data(), sizeof(int) * vb.size());
    if (times) memcpy(times, vt.data(), sizeof(int) * vt.size());
    if (mapping) memcpy(mapping, vm.data(), sizeof(int) * vm.size());
    return AI2B_OK;
}

// ---------------------------------------------------------------------------------------------
// Table compiler
// ---------------------------------------------------------------------------------------------
namespace {
struct Blob {
    std::vector<unsigned char> bytes;
    template <typename V>
    size_t add(const std::vector<V> &v)
    {
        size_t off = (bytes.size() + 255) & ~size_t(255);
        bytes.resize(off + std::max<size_t>(sizeof(V) * v.size(), 16));
        if (!v.empty()) memcpy(bytes.data() + off, v.data(), sizeof(V) * v.size());
        return off;
    }
};
}  // namespace

extern "C" int ai2b_mtp_program_create(int nm, int nb, const int *basic, int nt, const int *times, int ns,
                                       const int *mapping, int nmus, ai2b_mtp_program **out)
{
    AI2B_REQUIRE(out && basic && mapping && (times || nt == 0), AI2B_ERR_INVALID, "ai2b_mtp_program_create: NULL argument");
    AI2B_REQUIRE(nm > 0 && nb > 0 && nt >= 0 && ns > 0 && nb <= nm, AI2B_ERR_INVALID, "ai2b_mtp_program_create: bad counts");
    AI2B_REQUIRE(nm <= 65535, AI2B_ERR_UNSUPPORTED, "alpha_moments_count %d > 65535 (template level > 28?)", nm);
    AI2B_REQUIRE(nmus >= 1 && nmus <= MTP_MAX_MU, AI2B_ERR_UNSUPPORTED, "nmus %d outside 1..%d", nmus, MTP_MAX_MU);

    MtpProgramDev P;
    memset(&P, 0, sizeof(P));
    P.nm = nm; P.nb = nb; P.nt = nt; P.ns = ns; P.nmus = nmus;
    for (int m = 0; m < MTP_MAX_MU; m++) P.kmu[m] = -1;
    for (int i = 0; i < nb; i++) {
        const int *r = basic + 4 * i;
        AI2B_REQUIRE(r[0] >= 0 && r[0] < nmus && r[1] >= 0 && r[2] >= 0 && r[3] >= 0, AI2B_ERR_INVALID,
                     "alpha_index_basic row %d out of range", i);
        int k = r[1] + r[2] + r[3];
        AI2B_REQUIRE(k <= MTP_MAX_DEG, AI2B_ERR_UNSUPPORTED,
                     "basic moment %d has degree %d > %d (template levels above 20 are not supported)", i, k, MTP_MAX_DEG);
        P.kmu[r[0]] = std::max(P.kmu[r[0]], k);
        P.kmax = std::max(P.kmax, k);
    }
    P.doff[0] = 0;
    for (int m = 0; m < nmus; m++) P.doff[m + 1] = P.doff[m] + ncan(P.kmu[m]);
    for (int m = nmus; m < MTP_MAX_MU; m++) P.doff[m + 1] = P.doff[nmus];
    P.ndense = P.doff[nmus];

    // dense numbering and the gather table that turns adjoints of the basic moments into
    // polynomial coefficients {value, d/dux, d/duy, d/duz} per canonical monomial
    std::vector<int> basic_dense(nb);
    std::vector<int4> e4g(P.ndense, make_int4(-1, -1, -1, -1));
    std::vector<int> e4m(P.ndense, 0);
    for (int i = 0; i < nb; i++) {
        const int *r = basic + 4 * i;
        int d = P.doff[r[0]] + canon_index(r[1], r[2], r[3]);
        basic_dense[i] = d;
        AI2B_REQUIRE(e4g[d].x == -1, AI2B_ERR_UNSUPPORTED, "alpha_index_basic row %d duplicates an earlier row", i);
        e4g[d].x = i;
    }
    for (int m = 0; m < nmus; m++)
        for (int k = 0; k <= P.kmu[m]; k++)
            for (int q = 0; q < ndeg(k); q++) {
                Exp3 e = deg_exp(k, q);
                int d = P.doff[m] + ncan(k - 1) + q;
                e4m[d] = (e.x + 1) | ((e.y + 1) << 8) | ((e.z + 1) << 16);
                if (k < P.kmu[m]) {
                    e4g[d].y = e4g[P.doff[m] + canon_index(e.x + 1, e.y, e.z)].x;
                    e4g[d].z = e4g[P.doff[m] + canon_index(e.x, e.y + 1, e.z)].x;
                    e4g[d].w = e4g[P.doff[m] + canon_index(e.x, e.y, e.z + 1)].x;
                }
            }

    std::vector<int> dense_basic(P.ndense, -1);
    std::vector<int4> e4d(P.ndense, make_int4(-1, -1, -1, -1));
    for (int i = 0; i < nb; i++) dense_basic[basic_dense[i]] = i;
    for (int d = 0; d < P.ndense; d++) {
        auto dn = [&](int bi) { return bi >= 0 ? basic_dense[bi] : -1; };
        e4d[d] = make_int4(dn(e4g[d].x), dn(e4g[d].y), dn(e4g[d].z), dn(e4g[d].w));
    }

    // product rows: dependency depth, and the requirement that sources are final before use
    std::vector<int> depth(nm, 0), last_write(nm, -1);
    for (int t = 0; t < nt; t++) {
        const int *r = times + 4 * t;
        AI2B_REQUIRE(r[0] >= 0 && r[0] < nm && r[1] >= 0 && r[1] < nm && r[3] >= 0 && r[3] < nm, AI2B_ERR_INVALID,
                     "alpha_index_times row %d out of range", t);
        last_write[r[3]] = t;
    }
    for (int t = 0; t < nt; t++) {
        const int *r = times + 4 * t;
        AI2B_REQUIRE(last_write[r[0]] < t && last_write[r[1]] < t, AI2B_ERR_UNSUPPORTED,
                     "alpha_index_times row %d reads a moment that a later row still accumulates into", t);
        depth[r[3]] = std::max(depth[r[3]], 1 + std::max(depth[r[0]], depth[r[1]]));
    }
    for (int t = 0; t < nt; t++)
        AI2B_REQUIRE(depth[times[4 * t + 3]] > std::max(depth[times[4 * t]], depth[times[4 * t + 1]]), AI2B_ERR_UNSUPPORTED,
                     "alpha_index_times row %d: inconsistent dependency order", t);
    for (int m = 0; m < nm; m++) P.nlev = std::max(P.nlev, depth[m]);
    AI2B_REQUIRE(P.nlev <= MTP_MAX_LEV, AI2B_ERR_UNSUPPORTED, "product depth %d > %d", P.nlev, MTP_MAX_LEV);

    // forward: destinations by depth, rows contiguous per destination, heavy destinations first
    std::vector<std::vector<int>> rows_of(nm), occ_of(nm);
    for (int t = 0; t < nt; t++) {
        rows_of[times[4 * t + 3]].push_back(t);
        occ_of[times[4 * t]].push_back(2 * t);        // entry: this moment is `a`, other = b
        occ_of[times[4 * t + 1]].push_back(2 * t + 1);  // this moment is `b`, other = a
    }
    std::vector<int4> fwd_dst, rev_mom;
    std::vector<int> fwd_ab, rev_od;
    std::vector<float> fwd_mf, rev_mf;
    std::vector<double> fwd_md, rev_md;
    P.fwd_lev_off[0] = 0;
    for (int lev = 1; lev <= P.nlev; lev++) {
        std::vector<int> ds;
        for (int m = 0; m < nm; m++)
            if (depth[m] == lev && !rows_of[m].empty()) ds.push_back(m);
        std::stable_sort(ds.begin(), ds.end(), [&](int a, int b) { return rows_of[a].size() > rows_of[b].size(); });
        for (int m : ds) {
            int rb = (int)fwd_ab.size();
            for (int t : rows_of[m]) {
                fwd_ab.push_back(times[4 * t] | (times[4 * t + 1] << 16));
                fwd_mf.push_back((float)times[4 * t + 2]);
                fwd_md.push_back((double)times[4 * t + 2]);
            }
            fwd_dst.push_back(make_int4(m, rb, (int)fwd_ab.size(), 0));
        }
        P.fwd_lev_off[lev] = (int)fwd_dst.size();
    }
    for (int lev = P.nlev + 1; lev <= MTP_MAX_LEV; lev++) P.fwd_lev_off[lev] = P.fwd_lev_off[P.nlev];
    // reverse: sources by depth, deepest first; adjoint[m] += sum adjoint[dst] * mult * M[other]
    P.rev_lev_off[0] = 0;
    for (int k = 0; k < P.nlev; k++) {
        int lev = P.nlev - 1 - k;
        std::vector<int> ms;
        for (int m = 0; m < nm; m++)
            if (depth[m] == lev && !occ_of[m].empty()) ms.push_back(m);
        std::stable_sort(ms.begin(), ms.end(), [&](int a, int b) { return occ_of[a].size() > occ_of[b].size(); });
        for (int m : ms) {
            int eb = (int)rev_od.size();
            for (int o : occ_of[m]) {
                int t = o >> 1;
                int other = (o & 1) ? times[4 * t] : times[4 * t + 1];
                rev_od.push_back(other | (times[4 * t + 3] << 16));
                rev_mf.push_back((float)times[4 * t + 2]);
                rev_md.push_back((double)times[4 * t + 2]);
            }
            rev_mom.push_back(make_int4(m, eb, (int)rev_od.size(), 0));
        }
        P.rev_lev_off[k + 1] = (int)rev_mom.size();
    }
    for (int k = P.nlev + 1; k <= MTP_MAX_LEV; k++) P.rev_lev_off[k] = P.rev_lev_off[P.nlev];

    std::vector<int2> fwd_rows(fwd_ab.size()), rev_ents(rev_od.size());
    for (size_t i = 0; i < fwd_ab.size(); i++) { int bits; memcpy(&bits, &fwd_mf[i], 4); fwd_rows[i] = make_int2(fwd_ab[i], bits); }
    for (size_t i = 0; i < rev_od.size(); i++) { int bits; memcpy(&bits, &rev_mf[i], 4); rev_ents[i] = make_int2(rev_od[i], bits); }
    // flat streams (same row order as fwd_ab / rev_od)
    std::vector<int2> fwd_flat(fwd_ab.size()), rev_flat(rev_od.size());
    int maxmult = 0;
    for (int lev = 0; lev <= MTP_MAX_LEV; lev++) {
        const int di = P.fwd_lev_off[lev];
        P.fwd_lev_row[lev] = di < (int)fwd_dst.size() ? fwd_dst[di].y : (int)fwd_ab.size();
        const int mi = P.rev_lev_off[lev];
        P.rev_lev_row[lev] = mi < (int)rev_mom.size() ? rev_mom[mi].y : (int)rev_od.size();
    }
    for (const int4 &d : fwd_dst)
        for (int r = d.y; r < d.z; r++) {
            const int mult = (int)fwd_md[r];
            maxmult = std::max(maxmult, mult);
            fwd_flat[r] = make_int2(fwd_ab[r], (mult & 0xff) | ((r == d.z - 1) ? 0x100 : 0) | (d.x << 16));
        }
    for (const int4 &m : rev_mom)
        for (int r = m.y; r < m.z; r++) {
            const int mult = (int)rev_md[r];
            maxmult = std::max(maxmult, mult);
            rev_flat[r] = make_int2(rev_od[r], (mult & 0xff) | ((r == m.z - 1) ? 0x100 : 0) | (m.x << 16));
        }
    AI2B_REQUIRE(maxmult <= 255, AI2B_ERR_UNSUPPORTED, "product multiplier %d > 255", maxmult);
    for (int t = 0; t < nt; t++)
        AI2B_REQUIRE(times[4 * t + 2] >= 0, AI2B_ERR_UNSUPPORTED, "negative product multiplier in row %d", t);
    std::vector<int> map(mapping, mapping + ns);
    for (int s = 0; s < ns; s++)
        AI2B_REQUIRE(map[s] >= 0 && map[s] < nm, AI2B_ERR_INVALID, "alpha_moment_mapping[%d] out of range", s);

    // segment streams (see mtp_program.cuh)
    std::vector<int4> seg_hdr;
    std::vector<int2> seg_row;
    std::vector<int> seg_wseg, seg_wrow, seg_init;
    {
        std::vector<char> is_source(nm, 0), is_mapped(nm, 0);
        for (int t = 0; t < nt; t++) { is_source[times[4 * t]] = 1; is_source[times[4 * t + 1]] = 1; }
        for (int s = 0; s < ns; s++) is_mapped[mapping[s]] = 1;
        // moments whose adjoint is just their seed: scalars that are no operand of any product, and basic
        // moments nothing uses (seed 0); every other adjoint that is read is written by a gather phase
        for (int m = 0; m < nm; m++)
            if (!is_source[m] && (is_mapped[m] || m < nb)) seg_init.push_back(m);
        struct Row { int x, y, mult; };
        auto emit_phase = [&](const std::vector<std::pair<int, std::vector<Row>>> &moments) {
            // longest processing time first over the workers; a segment (rows of one multiplier) costs about as much as
            // two and a half of its rows (header, multiplier, final store)
            std::vector<long> cost(moments.size());
            for (size_t i = 0; i < moments.size(); i++) {
                std::vector<int> mults;
                for (const Row &r : moments[i].second) mults.push_back(r.mult);
                std::sort(mults.begin(), mults.end());
                const long nseg = (long)(std::unique(mults.begin(), mults.end()) - mults.begin());
                cost[i] = 2 * (long)moments[i].second.size() + 5 * nseg;
            }
            std::vector<size_t> order(moments.size());
            for (size_t i = 0; i < order.size(); i++) order[i] = i;
            std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) { return cost[a] > cost[b]; });
            std::vector<std::vector<size_t>> mine(MTP_SEG_WORKERS);
            std::vector<long> load(MTP_SEG_WORKERS, 0);
            for (size_t i : order) {
                int w = (int)(std::min_element(load.begin(), load.end()) - load.begin());
                mine[w].push_back(i);
                load[w] += cost[i];
            }
            for (int w = 0; w < MTP_SEG_WORKERS; w++) {
                seg_wseg.push_back((int)seg_hdr.size());
                seg_wrow.push_back((int)seg_row.size());
                for (size_t i : mine[w]) {
                    std::vector<Row> rows = moments[i].second;
                    std::stable_sort(rows.begin(), rows.end(), [](const Row &a, const Row &b) { return a.mult < b.mult; });
                    size_t r = 0;
                    bool first = true;
                    while (r < rows.size()) {
                        size_t e = r;
                        while (e < rows.size() && rows[e].mult == rows[r].mult) e++;
                        const double mult = (double)rows[r].mult;
                        long long bits;
                        memcpy(&bits, &mult, 8);
                        unsigned flags = (unsigned)(e - r) | (first ? 1u << 30 : 0u) | (e == rows.size() ? 1u << 31 : 0u);
                        seg_hdr.push_back(make_int4(moments[i].first * MTP_SEG_LD, (int)flags, (int)(bits & 0xffffffffll), (int)(bits >> 32)));
                        for (size_t k = r; k < e; k++) seg_row.push_back(make_int2(rows[k].x * MTP_SEG_LD, rows[k].y * MTP_SEG_LD));
                        first = false;
                        r = e;
                    }
                }
            }
            seg_wseg.push_back((int)seg_hdr.size());
        };
        for (int lev = 1; lev <= P.nlev; lev++) {
            std::vector<std::pair<int, std::vector<Row>>> moments;
            for (int m = 0; m < nm; m++)
                if (depth[m] == lev && !rows_of[m].empty()) {
                    std::vector<Row> rows;
                    for (int t : rows_of[m]) rows.push_back(Row{times[4 * t], times[4 * t + 1], times[4 * t + 2]});
                    moments.emplace_back(m, rows);
                }
            emit_phase(moments);
        }
        for (int k = 0; k < P.nlev; k++) {
            const int lev = P.nlev - 1 - k;
            std::vector<std::pair<int, std::vector<Row>>> moments;
            for (int m = 0; m < nm; m++)
                if (depth[m] == lev && !occ_of[m].empty()) {
                    std::vector<Row> rows;
                    for (int o : occ_of[m]) {
                        const int t = o >> 1;
                        const int other = (o & 1) ? times[4 * t] : times[4 * t + 1];
                        rows.push_back(Row{times[4 * t + 3], other, times[4 * t + 2]});
                    }
                    moments.emplace_back(m, rows);
                }
            emit_phase(moments);
        }
        for (const int4 &h : seg_hdr)
            AI2B_REQUIRE((h.y & 0x3fffffff) < (1 << 24), AI2B_ERR_UNSUPPORTED, "a product segment has too many rows");
    }
    P.nseg = (int)seg_hdr.size();
    P.nseg_rows = (int)seg_row.size();
    P.nseg_init = (int)seg_init.size();

    Blob blob;
    size_t o_sh = blob.add(seg_hdr), o_sr = blob.add(seg_row), o_sws = blob.add(seg_wseg), o_swr = blob.add(seg_wrow), o_si = blob.add(seg_init);
    size_t o_bd = blob.add(basic_dense), o_db = blob.add(dense_basic), o_e4d = blob.add(e4d), o_g = blob.add(e4g), o_m = blob.add(e4m), o_fd = blob.add(fwd_dst),
           o_fr = blob.add(fwd_ab), o_fmf = blob.add(fwd_mf), o_fmd = blob.add(fwd_md), o_rm = blob.add(rev_mom),
           o_re = blob.add(rev_od), o_rmf = blob.add(rev_mf), o_rmd = blob.add(rev_md), o_map = blob.add(map);
    size_t o_frow = blob.add(fwd_rows), o_rent = blob.add(rev_ents), o_ff = blob.add(fwd_flat), o_rf = blob.add(rev_flat);
    ai2b_mtp_program *prog = new ai2b_mtp_program;
    prog->blob_bytes = blob.bytes.size();
    prog->d_blob = nullptr;
    cudaError_t e = cudaGetDevice(&prog->device);
    if (e == cudaSuccess) e = cudaMalloc(&prog->d_blob, prog->blob_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(prog->d_blob, blob.bytes.data(), prog->blob_bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        set_error("ai2b_mtp_program_create: %s", cudaGetErrorString(e));
        if (prog->d_blob) cudaFree(prog->d_blob);
        delete prog;
        return AI2B_ERR_CUDA;
    }
    unsigned char *b = (unsigned char *)prog->d_blob;
    P.basic_dense = (const int *)(b + o_bd);
    P.dense_basic = (const int *)(b + o_db);
    P.e4d = (const int4 *)(b + o_e4d);
    P.e4g = (const int4 *)(b + o_g);
    P.e4m = (const int *)(b + o_m);
    P.fwd_dst = (const int4 *)(b + o_fd);
    P.fwd_ab = (const int *)(b + o_fr);
    P.fwd_mult_f = (const float *)(b + o_fmf);
    P.fwd_mult_d = (const double *)(b + o_fmd);
    P.rev_mom = (const int4 *)(b + o_rm);
    P.rev_od = (const int *)(b + o_re);
    P.rev_mult_f = (const float *)(b + o_rmf);
    P.rev_mult_d = (const double *)(b + o_rmd);
    P.map = (const int *)(b + o_map);
    P.fwd_rows = (const int2 *)(b + o_frow);
    P.rev_ents = (const int2 *)(b + o_rent);
    P.fwd_flat = (const int2 *)(b + o_ff);
    P.rev_flat = (const int2 *)(b + o_rf);
    P.seg_hdr = (const int4 *)(b + o_sh);
    P.seg_row = (const int2 *)(b + o_sr);
    P.seg_wseg = (const int *)(b + o_sws);
    P.seg_wrow = (const int *)(b + o_swr);
    P.seg_init = (const int *)(b + o_si);
    prog->dev = P;
    *out = prog;
    return AI2B_OK;
}

extern "C" void ai2b_mtp_program_destroy(ai2b_mtp_program *prog)
{
    if (!prog) return;
    if (prog->d_blob) cudaFree(prog->d_blob);
    delete prog;
}
