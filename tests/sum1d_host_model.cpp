// Host model of the summarised chain sum: the same passes as repdl_b200/csrc/sum1d.cu (tile sums,
// prediction scan, leaf classification, item plan, item emission, walk), run as plain loops on the
// CPU with the arithmetic of repdl_b200/csrc/sum1d_core.cuh, which the CUDA kernels include too.
// The CPU test-suite compiles this with g++ and compares its result bit for bit with the plain
// chain; it is how the algebra (summaries, orientation, ties, item skipping, fall-backs) is checked
// where no GPU is available.  Build: g++ -O2 -ffp-contract=off -shared -fPIC.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../repdl_b200/csrc/sum1d_core.cuh"

using namespace repdl_b200::s1;

namespace {

struct NodeRec {
    Summ pos;  // composed positive-orientation summary (smooth nodes)
    int sek, kind, count;
};
enum { N_SMOOTH = 0, N_MIXED = 1, N_RAW = 2 };

inline float elem(const float *x, int64_t n, int64_t i) { return i < n ? x[i] : 0.0f; }

// Codes and positive-orientation summaries of one node's leaves.
void classify_node(const float *x, int64_t n, int64_t node, const double *tile_sum, double pred, double rabs,
                   unsigned short *code, Summ *summ)
{
    double p_tile = pred;
    for (int t = 0; t < TILES_PER_NODE; t++) {
        double p = p_tile;
        for (int l = 0; l < 32; l++) {
            const int64_t e0 = node * NODE + (int64_t)t * TILE + (int64_t)l * LEAF;
            float v[LEAF];
            double ls = 0.0;
            for (int i = 0; i < LEAF; i++) {
                v[i] = elem(x, n, e0 + i);
                ls += (double)v[i];
            }
            const int sek = hyp_sign_exp(p);
            const Summ sm = leaf_summary(v, sek & 255);
            const int cls = classify_leaf(sm, sek, p, rabs);
            code[t * 32 + l] = (unsigned short)leaf_code(cls, sek);
            summ[t * 32 + l] = sm;
            p += ls;
        }
        p_tile += tile_sum[node * TILES_PER_NODE + t];
    }
}

}  // namespace

// stats[0..7]: items, runs, softs, leaves, hards, rawspans, failed runs, leaves walked with real adds;
// stats[8]: failed softs; stats[9]: mixed nodes
extern "C" float s1_model_sum(const float *x, int64_t n, float factor, int64_t *stats, int64_t cap_override)
{
    const int64_t nnodes = (n + NODE - 1) / NODE;
    std::vector<double> tile_sum(nnodes * TILES_PER_NODE), node_sum(nnodes), pred(nnodes), rabs(nnodes);
    for (int64_t nd = 0; nd < nnodes; nd++) {
        double ns = 0.0;
        for (int t = 0; t < TILES_PER_NODE; t++) {
            double ts = 0.0;
            for (int i = 0; i < TILE; i++) ts += (double)elem(x, n, nd * NODE + (int64_t)t * TILE + i);
            tile_sum[nd * TILES_PER_NODE + t] = ts;
            ns += ts;
        }
        node_sum[nd] = ns;
    }
    double run = 0.0, var = 0.0;
    for (int64_t nd = 0; nd < nnodes; nd++) {
        pred[nd] = run;
        const double a = fabs(run), b = fabs(run + node_sum[nd]);
        var += drift_variance(a > b ? a : b);
        rabs[nd] = DRIFT_SIGMAS * sqrt(var);
        run += node_sum[nd];
    }
    std::vector<NodeRec> rec(nnodes);
    std::vector<unsigned short> code(LEAVES_PER_NODE);
    std::vector<Summ> summ(LEAVES_PER_NODE);
    int64_t mixed = 0;
    for (int64_t nd = 0; nd < nnodes; nd++) {
        classify_node(x, n, nd, tile_sum.data(), pred[nd], rabs[nd], code.data(), summ.data());
        int count = 0;
        bool smooth = true;
        for (int i = 0; i < LEAVES_PER_NODE; i++) {
            count += leaf_item_count(code.data(), i);
            smooth &= code[i] == code[0] && code_class(code[i]) == C_ROBUST;
        }
        NodeRec r{};
        if (smooth) {
            Summ acc = summ[0];
            for (int i = 1; i < LEAVES_PER_NODE; i++) acc = summ_compose(acc, summ[i]);
            r = {acc, code_sek(code[0]), N_SMOOTH, 1};
        } else {
            r = {summ_invalid(), 0, N_MIXED, count};
            mixed++;
        }
        rec[nd] = r;
    }
    // plan.  Consecutive smooth nodes under one hypothesis are merged under a header item (K_SOFT
    // semantics: applied -> the nodes' own items are skipped); a merged stretch stays inside one of
    // the 1024 chunks of nodes that the GPU's planning threads own.
    const int64_t cap = cap_override > 0 ? cap_override : item_capacity(nnodes);
    std::vector<int64_t> off(nnodes);
    std::vector<Item> items;
    const int64_t per = (nnodes + 1023) / 1024;
    auto plan_merged = [&](bool write) {
        int64_t run = 0;
        for (int64_t lo = 0; lo < nnodes; lo += per) {
            const int64_t hi = lo + per < nnodes ? lo + per : nnodes;
            int64_t i = lo;
            while (i < hi) {
                if (rec[i].kind != N_SMOOTH) {
                    off[i] = run;
                    run += rec[i].count;
                    i++;
                    continue;
                }
                int64_t j = i + 1;
                Summ acc = rec[i].pos;
                while (j < hi && rec[j].kind == N_SMOOTH && rec[j].sek == rec[i].sek) {
                    acc = summ_compose(acc, rec[j].pos);
                    j++;
                }
                const int len = (int)(j - i);
                if (len >= 2) {
                    if (write)
                        items[run] = make_item(K_SOFT, acc, rec[i].sek, len, (int)(i * LEAVES_PER_NODE),
                                               len * LEAVES_PER_NODE);
                    run++;
                }
                for (int64_t k = i; k < j; k++) off[k] = run + (k - i);
                run += len;
                i = j;
            }
        }
        return run;
    };
    int64_t total = plan_merged(false);
    if (total <= cap) {
        items.resize(total);
        plan_merged(true);
    } else {
        // no merging; from the first node whose items would no longer fit, every node is raw
        int64_t o = 0, first_over = nnodes;
        for (int64_t nd = 0; nd < nnodes; nd++) {
            if (first_over == nnodes && o + rec[nd].count + (nnodes - nd - 1) > cap) first_over = nd;
            if (nd >= first_over) rec[nd].kind = N_RAW, rec[nd].count = 1;
            off[nd] = o;
            o += rec[nd].count;
        }
        total = o;
        if (total > cap) return 0.0f / 0.0f;  // cannot happen for cap >= nnodes
        items.resize(total);
    }
    for (int64_t nd = 0; nd < nnodes; nd++) {
        Item *out = items.data() + off[nd];
        const int leaf0 = (int)(nd * LEAVES_PER_NODE);
        if (rec[nd].kind == N_SMOOTH) {
            out[0] = make_item(K_RUN, rec[nd].pos, rec[nd].sek, 0, leaf0, LEAVES_PER_NODE);
        } else if (rec[nd].kind == N_RAW) {
            out[0] = make_item(K_RAWSPAN, summ_invalid(), 0, 0, leaf0, LEAVES_PER_NODE);
        } else {
            classify_node(x, n, nd, tile_sum.data(), pred[nd], rabs[nd], code.data(), summ.data());
            int k = 0;
            for (int i = 0; i < LEAVES_PER_NODE; i++) {
                leaf_emit_items(code.data(), summ.data(), i, leaf0, out + k);
                k += leaf_item_count(code.data(), i);
            }
            if (k != rec[nd].count) return 0.0f / 0.0f;
        }
    }
    // walk
    int64_t st[16] = {0};
    st[0] = total, st[9] = mixed;
    int bits = 0;  // +0.0f
    auto raw_span = [&](int64_t leaf, int64_t len) {
        float s = i2f(bits);
        for (int64_t e = leaf * LEAF; e < (leaf + len) * LEAF && e < n; e++) s = s + x[e];
        bits = f2i(s);
        st[7] += len;
    };
#ifdef S1_MODEL_EXPORT
    std::vector<int> entry(total, 0);
    std::vector<char> visited(total, 0);
#endif
    for (int64_t i = 0; i < total;) {
        const Item &it = items[i];
        const int kind = it.kind_skip & 255, skip = it.kind_skip >> 8;
        st[1 + kind]++;
#ifdef S1_MODEL_EXPORT
        entry[i] = bits, visited[i] = 1;
#endif
        if (kind <= K_LEAF) {
            if (item_apply(bits, it)) {
                i += 1 + (kind == K_SOFT ? skip : 0);
                continue;
            }
            if (kind == K_SOFT) {
                st[8]++;
                i++;
                continue;
            }
            if (kind == K_RUN) st[6]++;
        }
        raw_span(it.start, it.len);
        i++;
    }
#ifdef S1_MODEL_EXPORT
    // debugging aid: the item stream, the state each visited item was entered with, and the final state
    if (FILE *f = fopen(getenv("S1_MODEL_EXPORT_PATH") ? getenv("S1_MODEL_EXPORT_PATH") : "/dev/null", "wb")) {
        fwrite(&total, 8, 1, f);
        fwrite(&bits, 4, 1, f);
        fwrite(items.data(), sizeof(Item), total, f);
        fwrite(entry.data(), 4, total, f);
        fwrite(visited.data(), 1, total, f);
        fclose(f);
    }
#endif
    if (stats)
        for (int k = 0; k < 10; k++) stats[k] = st[k];
    return factor * i2f(bits);
}
