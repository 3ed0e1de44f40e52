// Both multi-GPU splits of the structure2vec inference path from a plain C++ host: one process, one host thread
// per GPU, nothing but the C ABI of include/s2v_b200.h and the CUDA runtime for device memory.
//
//   s2v_multi_gpu shard <batch.bin> <out.bin> [--gpus N] [--iters K]
//       A batch of small graphs sharded by graph: contiguous graph ranges balanced by node count, every GPU runs
//       the whole classifier on its range (s2v_forward_f32) with a replica of the weights, and the only exchange is
//       the final s2v_gather_logits.  batch.bin is the format of s2v_mean_field (int32 header {G, N, E, F, d, L,
//       hidden, C}, nodes_per_graph, edge_src, edge_dst, tags, four weight matrices).
//       out.bin: logits[G*C] (fp32), pred[G] (int32) as gathered on rank 0.
//
//   s2v_multi_gpu giant <graph.bin> <out.bin> [--gpus N] [--levels L] [--chunks C] [--iters K] [--exchange referenced]
//       One graph partitioned by rows: GPU p owns rows [p*N/P, (p+1)*N/P) of A and of H; a level is the fused level
//       kernel on the local rows (all of H as the gather source) and one all-gather of the new rows.  The local rows
//       are cut into C blocks and block k is exchanged (s2v_allgather_rows_f32, in place, on a second stream) while
//       block k+1 is computed.  H is stored block-major ([block][rank][rows of the block][d]) so that every exchange
//       is one contiguous range; the column indices are renumbered to that layout once.
//       With --exchange referenced every GPU fetches only the rows of H that its own rows name: its table is
//       [own rows | referenced remote rows in ascending order]; per block the owner packs the rows each peer asked for
//       (s2v_input_proj_onehot_f32 is the row lookup) and one s2v_exchange_rows_f32 drops them into the peers' tables.
//       graph.bin: int64 header {N, nnz, d}, row_ptr int64[N+1], col_idx int32[nnz], H0 fp32[N*d], W fp32[d*d].
//       out.bin: H_L fp32[N*d] in row order.
//
// Prints one line per run: "<mode> gpus <P> ms_per_iter <t>" (device time of the slowest GPU, CUDA events).
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "s2v_b200.h"

namespace
{

[[noreturn]] void die(const std::string& what)
{
    fprintf(stderr, "s2v_multi_gpu: %s\n", what.c_str());
    exit(1);
}
void ok_cuda(cudaError_t e, const char* what)
{
    if (e != cudaSuccess) die(std::string(what) + ": " + cudaGetErrorString(e));
}
void ok_s2v(int rc, s2v_ctx* ctx, const char* what)
{
    if (rc != S2V_OK) die(std::string(what) + ": " + s2v_status_str(rc) + " (" + s2v_last_error(ctx) + ")");
}
void ok_comm(int rc, s2v_comm* comm, const char* what)
{
    if (rc != S2V_OK) die(std::string(what) + ": " + s2v_status_str(rc) + " (" + s2v_comm_last_error(comm) + ")");
}

template <typename T>
void read_vec(FILE* f, std::vector<T>& v, size_t n)
{
    v.resize(n);
    if (n && fread(v.data(), sizeof(T), n, f) != n) die("input file is truncated");
}
template <typename T>
T* to_device(const std::vector<T>& v)
{
    T* p = nullptr;
    ok_cuda(cudaMalloc(&p, std::max<size_t>(v.size(), 1) * sizeof(T)), "cudaMalloc");
    if (!v.empty()) ok_cuda(cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
    return p;
}

// all host threads meet here between phases
struct SpinBarrier {
    explicit SpinBarrier(int n) : n_(n) {}
    void wait()
    {
        const int gen = gen_.load();
        if (count_.fetch_add(1) + 1 == n_) {
            count_.store(0);
            gen_.fetch_add(1);
        } else {
            while (gen_.load() == gen) std::this_thread::yield();
        }
    }
    int n_;
    std::atomic<int> count_{0}, gen_{0};
};

int arg_int(int argc, char** argv, const char* name, int dflt)
{
    for (int i = 0; i + 1 < argc; ++i)
        if (!strcmp(argv[i], name)) return atoi(argv[i + 1]);
    return dflt;
}

// ------------------------------------------------------------------ shard by graph
struct Batch {
    int G, N, E, F, d, L, hidden, C;
    std::vector<int32_t> nodes_per_graph, edge_src, edge_dst, tags;
    std::vector<float> w_n2l, p_node_conv, h1_weight, h2_weight;
};

Batch load_batch(const char* path)
{
    FILE* f = fopen(path, "rb");
    if (!f) die(std::string("cannot open ") + path);
    int h[8];
    if (fread(h, sizeof(int), 8, f) != 8) die("batch file has no header");
    Batch b;
    b.G = h[0]; b.N = h[1]; b.E = h[2]; b.F = h[3]; b.d = h[4]; b.L = h[5]; b.hidden = h[6]; b.C = h[7];
    read_vec(f, b.nodes_per_graph, b.G);
    read_vec(f, b.edge_src, b.E);
    read_vec(f, b.edge_dst, b.E);
    read_vec(f, b.tags, b.N);
    read_vec(f, b.w_n2l, (size_t)b.F * b.d);
    read_vec(f, b.p_node_conv, (size_t)b.d * b.d);
    read_vec(f, b.h1_weight, (size_t)b.d * b.hidden);
    read_vec(f, b.h2_weight, (size_t)b.hidden * b.C);
    fclose(f);
    return b;
}

// contiguous graph ranges with near-equal node totals: rank r starts after the graph that reaches r/P of the nodes
std::vector<int> graph_cuts(const std::vector<int32_t>& nodes_per_graph, int world)
{
    const int G = (int)nodes_per_graph.size();
    std::vector<long long> cum(G);
    long long run = 0;
    for (int g = 0; g < G; ++g) cum[g] = (run += nodes_per_graph[g]);
    std::vector<int> cuts(world + 1, 0);
    for (int r = 1; r < world; ++r) {
        const double target = (double)run * r / world;
        const int idx = (int)(std::lower_bound(cum.begin(), cum.end(), target, [](long long c, double t) { return (double)c < t; }) - cum.begin());
        cuts[r] = std::min(std::max(idx + 1, cuts[r - 1]), G);
    }
    cuts[world] = G;
    for (int r = 1; r <= world; ++r) cuts[r] = std::max(cuts[r], cuts[r - 1]);
    return cuts;
}

int run_shard(const char* in_path, const char* out_path, int P, int iters)
{
    const Batch b = load_batch(in_path);
    const std::vector<int> cuts = graph_cuts(b.nodes_per_graph, P);
    std::vector<long long> node_off(b.G + 1, 0);
    for (int g = 0; g < b.G; ++g) node_off[g + 1] = node_off[g] + b.nodes_per_graph[g];
    std::vector<int> devs(P);
    for (int p = 0; p < P; ++p) devs[p] = p;
    std::vector<s2v_comm*> comms(P, nullptr);
    ok_comm(s2v_comm_create(P, devs.data(), comms.data()), nullptr, "s2v_comm_create");
    std::vector<int64_t> counts(P);
    for (int p = 0; p < P; ++p) counts[p] = cuts[p + 1] - cuts[p];
    std::vector<float> logits_all((size_t)b.G * b.C);
    std::vector<int32_t> pred_all(b.G);
    std::vector<float> ms(P, 0.f);
    SpinBarrier barrier(P);

    auto worker = [&](int p) {
        ok_cuda(cudaSetDevice(devs[p]), "cudaSetDevice");
        s2v_ctx* ctx = nullptr;
        ok_s2v(s2v_ctx_create(devs[p], &ctx), nullptr, "s2v_ctx_create");
        // this rank's graphs as a batch of its own: node ids rebased, edges of the range in their original order
        const int g_lo = cuts[p], g_hi = cuts[p + 1];
        const long long n_lo = node_off[g_lo], n_hi = node_off[g_hi];
        const int64_t G = g_hi - g_lo, N = n_hi - n_lo;
        std::vector<int32_t> es, ed, graph_ptr(G + 1), tags(b.tags.begin() + n_lo, b.tags.begin() + n_hi);
        for (int e = 0; e < b.E; ++e)
            if (b.edge_src[e] >= n_lo && b.edge_src[e] < n_hi) {
                es.push_back((int32_t)(b.edge_src[e] - n_lo));
                ed.push_back((int32_t)(b.edge_dst[e] - n_lo));
            }
        int32_t max_nodes = 0;
        for (int64_t g = 0; g <= G; ++g) graph_ptr[g] = (int32_t)(node_off[g_lo + g] - n_lo);
        for (int64_t g = 0; g < G; ++g) max_nodes = std::max(max_nodes, graph_ptr[g + 1] - graph_ptr[g]);
        const int64_t E = (int64_t)es.size();
        std::vector<int32_t> row_ptr(N + 1), col_idx(std::max<int64_t>(E, 1));
        if (s2v_build_n2n_csr_host(N, E, es.data(), ed.data(), 0, row_ptr.data(), col_idx.data(), nullptr) != S2V_OK) die("CSR construction failed");
        col_idx.resize(E);

        s2v_model model{};
        model.num_feat = b.F; model.d = b.d; model.levels = b.L; model.hidden = b.hidden; model.num_class = b.C;
        model.w_n2l = to_device(b.w_n2l);
        model.p_node_conv = to_device(b.p_node_conv);
        model.h1_weight = to_device(b.h1_weight);
        model.h2_weight = to_device(b.h2_weight);
        s2v_batch batch{};
        batch.num_graphs = G; batch.num_nodes = N; batch.num_edges = E;
        batch.n2n_row_ptr = to_device(row_ptr);
        batch.n2n_col_idx = to_device(col_idx);
        batch.graph_ptr = to_device(graph_ptr);
        batch.tags = to_device(tags);
        batch.max_graph_nodes = max_nodes;
        const size_t ws_bytes = s2v_forward_workspace_bytes(N, G, b.d);
        void* ws = nullptr;
        float *logits = nullptr, *d_logits_all = nullptr;
        int32_t *pred = nullptr, *d_pred_all = nullptr;
        ok_cuda(cudaMalloc(&ws, ws_bytes), "cudaMalloc workspace");
        ok_cuda(cudaMalloc(&logits, sizeof(float) * std::max<int64_t>(G, 1) * b.C), "cudaMalloc");
        ok_cuda(cudaMalloc(&pred, sizeof(int32_t) * std::max<int64_t>(G, 1)), "cudaMalloc");
        ok_cuda(cudaMalloc(&d_logits_all, sizeof(float) * (size_t)b.G * b.C), "cudaMalloc");
        ok_cuda(cudaMalloc(&d_pred_all, sizeof(int32_t) * (size_t)b.G), "cudaMalloc");
        s2v_stream st = s2v_ctx_stream(ctx);
        cudaEvent_t e0, e1;
        ok_cuda(cudaEventCreate(&e0), "cudaEventCreate");
        ok_cuda(cudaEventCreate(&e1), "cudaEventCreate");
        float total = 0.f;
        for (int it = 0; it < iters + 1; ++it) {   // the first iteration is a warm-up
            barrier.wait();
            ok_cuda(cudaEventRecord(e0, (cudaStream_t)st), "cudaEventRecord");
            if (G > 0) ok_s2v(s2v_forward_f32(ctx, st, &model, &batch, ws, ws_bytes, logits, nullptr, pred, nullptr), ctx, "s2v_forward_f32");
            ok_comm(s2v_gather_logits(comms[p], st, counts.data(), b.C, logits, pred, d_logits_all, d_pred_all), comms[p], "s2v_gather_logits");
            ok_cuda(cudaEventRecord(e1, (cudaStream_t)st), "cudaEventRecord");
            ok_s2v(s2v_stream_status(ctx, st), ctx, "device status");
            float t = 0.f;
            ok_cuda(cudaEventElapsedTime(&t, e0, e1), "cudaEventElapsedTime");
            if (it > 0) total += t;
        }
        ms[p] = total / iters;
        if (p == 0) {
            ok_cuda(cudaMemcpy(logits_all.data(), d_logits_all, sizeof(float) * logits_all.size(), cudaMemcpyDeviceToHost), "cudaMemcpy");
            ok_cuda(cudaMemcpy(pred_all.data(), d_pred_all, sizeof(int32_t) * pred_all.size(), cudaMemcpyDeviceToHost), "cudaMemcpy");
        }
        barrier.wait();
        s2v_ctx_destroy(ctx);
    };
    std::vector<std::thread> threads;
    for (int p = 0; p < P; ++p) threads.emplace_back(worker, p);
    for (auto& t : threads) t.join();
    for (int p = 0; p < P; ++p) s2v_comm_destroy(comms[p]);
    FILE* f = fopen(out_path, "wb");
    if (!f) die(std::string("cannot write ") + out_path);
    fwrite(logits_all.data(), sizeof(float), logits_all.size(), f);
    fwrite(pred_all.data(), sizeof(int32_t), pred_all.size(), f);
    fclose(f);
    printf("shard gpus %d ms_per_iter %.4f\n", P, *std::max_element(ms.begin(), ms.end()));
    return 0;
}

// ------------------------------------------------------------------ giant graph, partitioned by rows
int run_giant_referenced(int64_t N, int d, const std::vector<int64_t>& row_ptr, const std::vector<int32_t>& col_idx,
                         const std::vector<float>& H0, const std::vector<float>& W, const char* out_path, int P, int levels, int chunks,
                         int iters);

int run_giant(const char* in_path, const char* out_path, int P, int levels, int chunks, int iters, bool referenced)
{
    FILE* f = fopen(in_path, "rb");
    if (!f) die(std::string("cannot open ") + in_path);
    int64_t h[3];
    if (fread(h, sizeof(int64_t), 3, f) != 3) die("graph file has no header");
    const int64_t N = h[0], nnz = h[1];
    const int d = (int)h[2];
    std::vector<int64_t> row_ptr;
    std::vector<int32_t> col_idx;
    std::vector<float> H0, W;
    read_vec(f, row_ptr, (size_t)N + 1);
    read_vec(f, col_idx, (size_t)nnz);
    read_vec(f, H0, (size_t)N * d);
    read_vec(f, W, (size_t)d * d);
    fclose(f);
    if (N % P) die("the number of rows must divide over the GPUs (pad the graph with isolated nodes)");
    if (referenced) return run_giant_referenced(N, d, row_ptr, col_idx, H0, W, out_path, P, levels, chunks, iters);
    const int64_t rows = N / P;
    chunks = (int)std::max<int64_t>(1, std::min<int64_t>(chunks, rows));
    std::vector<int64_t> edge(chunks + 1);
    for (int k = 0; k <= chunks; ++k) edge[k] = rows * k / chunks;
    // position of global row (r * rows + i) in the block-major layout [block][rank][rows of the block]
    auto position = [&](int64_t g) -> int64_t {
        const int64_t r = g / rows, i = g % rows;
        const int k = (int)(std::upper_bound(edge.begin(), edge.end(), i) - edge.begin()) - 1;
        return P * edge[k] + r * (edge[k + 1] - edge[k]) + (i - edge[k]);
    };
    std::vector<int> devs(P);
    for (int p = 0; p < P; ++p) devs[p] = p;
    std::vector<s2v_comm*> comms(P, nullptr);
    ok_comm(s2v_comm_create(P, devs.data(), comms.data()), nullptr, "s2v_comm_create");
    std::vector<float> out((size_t)N * d);
    std::vector<float> ms(P, 0.f);
    SpinBarrier barrier(P);

    auto worker = [&](int p) {
        ok_cuda(cudaSetDevice(devs[p]), "cudaSetDevice");
        s2v_ctx* ctx = nullptr;
        ok_s2v(s2v_ctx_create(devs[p], &ctx), nullptr, "s2v_ctx_create");
        // my rows of A: row offsets rebased per block, columns renumbered to the block-major layout
        const int64_t r_lo = p * rows;
        std::vector<int32_t> cols((size_t)(row_ptr[r_lo + rows] - row_ptr[r_lo]));
        for (size_t t = 0; t < cols.size(); ++t) cols[t] = (int32_t)position(col_idx[row_ptr[r_lo] + t]);
        std::vector<int64_t> rp((size_t)rows + chunks);   // per block: rows_k + 1 offsets starting at 0
        std::vector<int64_t> rp_at(chunks), nnz_at(chunks);
        {
            size_t w = 0;
            for (int k = 0; k < chunks; ++k) {
                rp_at[k] = (int64_t)w;
                const int64_t b0 = row_ptr[r_lo + edge[k]];
                nnz_at[k] = b0 - row_ptr[r_lo];
                for (int64_t i = edge[k]; i <= edge[k + 1]; ++i) rp[w++] = row_ptr[r_lo + i] - b0;
            }
        }
        int64_t* d_rp = to_device(rp);
        int32_t* d_cols = to_device(cols);
        float* d_W = to_device(W);
        // full[0] holds H0 and is never written; the levels alternate between full[1] and full[2]
        float* full[3];
        for (int i = 0; i < 3; ++i) ok_cuda(cudaMalloc(&full[i], sizeof(float) * (size_t)N * d), "cudaMalloc H");
        {
            std::vector<float> h0_layout((size_t)N * d);
            for (int64_t g = 0; g < N; ++g) memcpy(&h0_layout[(size_t)position(g) * d], &H0[(size_t)g * d], sizeof(float) * d);
            ok_cuda(cudaMemcpy(full[0], h0_layout.data(), sizeof(float) * (size_t)N * d, cudaMemcpyHostToDevice), "cudaMemcpy H0");
        }
        cudaStream_t compute = (cudaStream_t)s2v_ctx_stream(ctx), exchange;
        ok_cuda(cudaStreamCreateWithFlags(&exchange, cudaStreamNonBlocking), "cudaStreamCreate");
        std::vector<cudaEvent_t> computed(chunks), gathered(chunks);
        for (int k = 0; k < chunks; ++k) {
            ok_cuda(cudaEventCreateWithFlags(&computed[k], cudaEventDisableTiming), "cudaEventCreate");
            ok_cuda(cudaEventCreateWithFlags(&gathered[k], cudaEventDisableTiming), "cudaEventCreate");
        }
        cudaEvent_t e0, e1;
        ok_cuda(cudaEventCreate(&e0), "cudaEventCreate");
        ok_cuda(cudaEventCreate(&e1), "cudaEventCreate");
        float total = 0.f;
        int last = 0;
        for (int it = 0; it < iters + 1; ++it) {
            barrier.wait();
            ok_cuda(cudaEventRecord(e0, compute), "cudaEventRecord");
            int cur = 0;
            for (int lv = 0; lv < levels; ++lv) {
                const int nxt = cur != 1 ? 1 : 2;
                for (int k = 0; k < chunks; ++k) {
                    const int64_t rk = edge[k + 1] - edge[k];
                    float* region = full[nxt] + (size_t)P * edge[k] * d;          // block k of all ranks, contiguous
                    float* piece = region + (size_t)p * rk * d;                   // my rows of block k
                    ok_s2v(s2v_level_rp64_f32(ctx, compute, rk, N, d, d_rp + rp_at[k], d_cols + nnz_at[k], nullptr, full[cur], d_W, nullptr, piece),
                           ctx, "s2v_level_rp64_f32");
                    ok_cuda(cudaEventRecord(computed[k], compute), "cudaEventRecord");
                    ok_cuda(cudaStreamWaitEvent(exchange, computed[k], 0), "cudaStreamWaitEvent");
                    ok_comm(s2v_allgather_rows_f32(comms[p], exchange, rk, d, piece, region), comms[p], "s2v_allgather_rows_f32");
                    ok_cuda(cudaEventRecord(gathered[k], exchange), "cudaEventRecord");
                }
                for (int k = 0; k < chunks; ++k) ok_cuda(cudaStreamWaitEvent(compute, gathered[k], 0), "cudaStreamWaitEvent");   // the next level reads every row
                cur = nxt;
            }
            last = cur;
            ok_cuda(cudaEventRecord(e1, compute), "cudaEventRecord");
            ok_s2v(s2v_stream_status(ctx, compute), ctx, "device status");
            float t = 0.f;
            ok_cuda(cudaEventElapsedTime(&t, e0, e1), "cudaEventElapsedTime");
            if (it > 0) total += t;
        }
        ms[p] = total / iters;
        // my rows of H_L, back in row order
        std::vector<float> mine((size_t)rows * d);
        for (int k = 0; k < chunks; ++k) {
            const int64_t rk = edge[k + 1] - edge[k];
            ok_cuda(cudaMemcpy(&mine[(size_t)edge[k] * d], full[last] + ((size_t)P * edge[k] + (size_t)p * rk) * d, sizeof(float) * (size_t)rk * d,
                               cudaMemcpyDeviceToHost), "cudaMemcpy");
        }
        memcpy(&out[(size_t)r_lo * d], mine.data(), sizeof(float) * mine.size());
        barrier.wait();
        s2v_ctx_destroy(ctx);
    };
    std::vector<std::thread> threads;
    for (int p = 0; p < P; ++p) threads.emplace_back(worker, p);
    for (auto& t : threads) t.join();
    for (int p = 0; p < P; ++p) s2v_comm_destroy(comms[p]);
    FILE* fo = fopen(out_path, "wb");
    if (!fo) die(std::string("cannot write ") + out_path);
    fwrite(out.data(), sizeof(float), out.size(), fo);
    fclose(fo);
    printf("giant gpus %d ms_per_iter %.4f\n", P, *std::max_element(ms.begin(), ms.end()));
    return 0;
}

// The same levels with every GPU fetching only the rows of H its own rows reference.
int run_giant_referenced(int64_t N, int d, const std::vector<int64_t>& row_ptr, const std::vector<int32_t>& col_idx,
                         const std::vector<float>& H0, const std::vector<float>& W, const char* out_path, int P, int levels, int chunks,
                         int iters)
{
    const int64_t rows = N / P;
    chunks = (int)std::max<int64_t>(1, std::min<int64_t>(chunks, rows));
    std::vector<int64_t> edge(chunks + 1);
    for (int k = 0; k <= chunks; ++k) edge[k] = rows * k / chunks;
    std::vector<int> devs(P);
    for (int p = 0; p < P; ++p) devs[p] = p;
    std::vector<s2v_comm*> comms(P, nullptr);
    ok_comm(s2v_comm_create(P, devs.data(), comms.data()), nullptr, "s2v_comm_create");
    std::vector<float> out((size_t)N * d);
    std::vector<float> ms(P, 0.f);
    std::vector<std::vector<int64_t>> needs(P);   // needs[p]: the remote rows GPU p references, ascending (shared by the threads)
    SpinBarrier barrier(P);

    auto worker = [&](int p) {
        ok_cuda(cudaSetDevice(devs[p]), "cudaSetDevice");
        s2v_ctx* ctx = nullptr;
        ok_s2v(s2v_ctx_create(devs[p], &ctx), nullptr, "s2v_ctx_create");
        const int64_t r_lo = p * rows;
        const int64_t my_nnz = row_ptr[r_lo + rows] - row_ptr[r_lo];
        {   // which remote rows do my rows name?
            std::vector<char> mark((size_t)N, 0);
            for (int64_t t = 0; t < my_nnz; ++t) mark[(size_t)col_idx[row_ptr[r_lo] + t]] = 1;
            for (int64_t g = 0; g < N; ++g)
                if (mark[(size_t)g] && (g < r_lo || g >= r_lo + rows)) needs[p].push_back(g);
        }
        barrier.wait();   // every GPU's list is known to every thread from here on
        const std::vector<int64_t>& need = needs[p];
        const int64_t n_need = (int64_t)need.size(), n_table = rows + n_need;
        auto position = [&](int64_t g) -> int64_t {   // own rows first, then the referenced remote rows
            if (g >= r_lo && g < r_lo + rows) return g - r_lo;
            return rows + (std::lower_bound(need.begin(), need.end(), g) - need.begin());
        };
        std::vector<int32_t> cols((size_t)my_nnz);
        for (size_t t = 0; t < cols.size(); ++t) cols[t] = (int32_t)position(col_idx[row_ptr[r_lo] + t]);
        std::vector<int64_t> rp((size_t)rows + chunks), rp_at(chunks), nnz_at(chunks);
        {
            size_t w = 0;
            for (int k = 0; k < chunks; ++k) {
                rp_at[k] = (int64_t)w;
                const int64_t b0 = row_ptr[r_lo + edge[k]];
                nnz_at[k] = b0 - row_ptr[r_lo];
                for (int64_t i = edge[k]; i <= edge[k + 1]; ++i) rp[w++] = row_ptr[r_lo + i] - b0;
            }
        }
        // per block: what I receive from every owner (a range of `need`), and what every peer asked of my block
        std::vector<std::vector<int64_t>> recv_off(chunks, std::vector<int64_t>(P, 0)), recv_cnt(chunks, std::vector<int64_t>(P, 0)),
            send_off(chunks, std::vector<int64_t>(P + 1, 0));
        std::vector<std::vector<int32_t>> send_idx(chunks);
        size_t max_send = 1;
        for (int k = 0; k < chunks; ++k) {
            for (int s = 0; s < P; ++s) {
                if (s == p) continue;
                const auto a = std::lower_bound(need.begin(), need.end(), s * rows + edge[k]);
                const auto b = std::lower_bound(need.begin(), need.end(), s * rows + edge[k + 1]);
                recv_off[k][s] = rows + (a - need.begin());
                recv_cnt[k][s] = b - a;
            }
            for (int t = 0; t < P; ++t) {
                send_off[k][t + 1] = send_off[k][t];
                if (t == p) continue;
                const auto a = std::lower_bound(needs[t].begin(), needs[t].end(), r_lo + edge[k]);
                const auto b = std::lower_bound(needs[t].begin(), needs[t].end(), r_lo + edge[k + 1]);
                for (auto it = a; it != b; ++it) send_idx[k].push_back((int32_t)(*it - r_lo));
                send_off[k][t + 1] += b - a;
            }
            max_send = std::max(max_send, send_idx[k].size());
        }
        int64_t* d_rp = to_device(rp);
        int32_t* d_cols = to_device(cols);
        float* d_W = to_device(W);
        std::vector<int32_t*> d_send_idx(chunks, nullptr);
        for (int k = 0; k < chunks; ++k)
            if (!send_idx[k].empty()) d_send_idx[k] = to_device(send_idx[k]);
        float* sendbuf = nullptr;
        ok_cuda(cudaMalloc(&sendbuf, sizeof(float) * max_send * d), "cudaMalloc send buffer");
        // table[0] holds H0 (own rows + the referenced remote rows, taken from the host copy) and is never written
        float* table[3];
        for (int i = 0; i < 3; ++i) ok_cuda(cudaMalloc(&table[i], sizeof(float) * (size_t)n_table * d), "cudaMalloc H");
        {
            std::vector<float> h0((size_t)n_table * d);
            memcpy(h0.data(), &H0[(size_t)r_lo * d], sizeof(float) * (size_t)rows * d);
            for (int64_t i = 0; i < n_need; ++i) memcpy(&h0[(size_t)(rows + i) * d], &H0[(size_t)need[i] * d], sizeof(float) * d);
            ok_cuda(cudaMemcpy(table[0], h0.data(), sizeof(float) * h0.size(), cudaMemcpyHostToDevice), "cudaMemcpy H0");
        }
        cudaStream_t compute = (cudaStream_t)s2v_ctx_stream(ctx), exchange;
        ok_cuda(cudaStreamCreateWithFlags(&exchange, cudaStreamNonBlocking), "cudaStreamCreate");
        std::vector<cudaEvent_t> computed(chunks), landed(chunks);
        for (int k = 0; k < chunks; ++k) {
            ok_cuda(cudaEventCreateWithFlags(&computed[k], cudaEventDisableTiming), "cudaEventCreate");
            ok_cuda(cudaEventCreateWithFlags(&landed[k], cudaEventDisableTiming), "cudaEventCreate");
        }
        cudaEvent_t e0, e1;
        ok_cuda(cudaEventCreate(&e0), "cudaEventCreate");
        ok_cuda(cudaEventCreate(&e1), "cudaEventCreate");
        float total = 0.f;
        int last = 0;
        for (int it = 0; it < iters + 1; ++it) {
            barrier.wait();
            ok_cuda(cudaEventRecord(e0, compute), "cudaEventRecord");
            int cur = 0;
            for (int lv = 0; lv < levels; ++lv) {
                const int nxt = cur != 1 ? 1 : 2;
                for (int k = 0; k < chunks; ++k) {
                    const int64_t rk = edge[k + 1] - edge[k];
                    float* piece = table[nxt] + (size_t)edge[k] * d;   // my rows of block k, in place in my table
                    ok_s2v(s2v_level_rp64_f32(ctx, compute, rk, n_table, d, d_rp + rp_at[k], d_cols + nnz_at[k], nullptr, table[cur], d_W, nullptr,
                                              piece), ctx, "s2v_level_rp64_f32");
                    ok_cuda(cudaEventRecord(computed[k], compute), "cudaEventRecord");
                    ok_cuda(cudaStreamWaitEvent(exchange, computed[k], 0), "cudaStreamWaitEvent");
                    const int64_t n_send = send_off[k][P];
                    if (n_send > 0)   // the rows of this block that the peers asked for, packed peer by peer
                        ok_s2v(s2v_input_proj_onehot_f32(ctx, exchange, n_send, (int)rows, d, d_send_idx[k], table[nxt], sendbuf, nullptr), ctx,
                               "s2v_input_proj_onehot_f32 (row lookup)");
                    ok_comm(s2v_exchange_rows_f32(comms[p], exchange, d, sendbuf, send_off[k].data(), table[nxt], recv_off[k].data(),
                                                  recv_cnt[k].data()), comms[p], "s2v_exchange_rows_f32");
                    ok_cuda(cudaEventRecord(landed[k], exchange), "cudaEventRecord");
                }
                for (int k = 0; k < chunks; ++k) ok_cuda(cudaStreamWaitEvent(compute, landed[k], 0), "cudaStreamWaitEvent");   // the next level reads the whole table
                cur = nxt;
            }
            last = cur;
            ok_cuda(cudaEventRecord(e1, compute), "cudaEventRecord");
            ok_s2v(s2v_stream_status(ctx, compute), ctx, "device status");
            ok_s2v(s2v_stream_status(ctx, exchange), ctx, "device status (exchange stream)");
            float t = 0.f;
            ok_cuda(cudaEventElapsedTime(&t, e0, e1), "cudaEventElapsedTime");
            if (it > 0) total += t;
        }
        ms[p] = total / iters;
        ok_cuda(cudaMemcpy(&out[(size_t)r_lo * d], table[last], sizeof(float) * (size_t)rows * d, cudaMemcpyDeviceToHost), "cudaMemcpy");
        barrier.wait();
        s2v_ctx_destroy(ctx);
    };
    std::vector<std::thread> threads;
    for (int p = 0; p < P; ++p) threads.emplace_back(worker, p);
    for (auto& t : threads) t.join();
    for (int p = 0; p < P; ++p) s2v_comm_destroy(comms[p]);
    FILE* fo = fopen(out_path, "wb");
    if (!fo) die(std::string("cannot write ") + out_path);
    fwrite(out.data(), sizeof(float), out.size(), fo);
    fclose(fo);
    int64_t need_total = 0;
    for (int p = 0; p < P; ++p) need_total += (int64_t)needs[p].size();
    printf("giant gpus %d ms_per_iter %.4f referenced_remote_rows %.4f\n", P, *std::max_element(ms.begin(), ms.end()),
           P > 1 ? (double)need_total / ((double)P * (double)(N - rows)) : 0.0);
    return 0;
}

}  // namespace

int main(int argc, char** argv)
{
    if (argc < 4) die("usage: s2v_multi_gpu shard|giant <in.bin> <out.bin> [--gpus N] [--iters K] [--levels L] [--chunks C] [--exchange referenced]");
    int have = 0;
    if (cudaGetDeviceCount(&have) != cudaSuccess || have == 0) die("no CUDA device");
    const int P = arg_int(argc, argv, "--gpus", 1);
    if (P < 1 || P > have) die("--gpus exceeds the devices present");
    const int iters = std::max(1, arg_int(argc, argv, "--iters", 3));
    if (!strcmp(argv[1], "shard")) return run_shard(argv[2], argv[3], P, iters);
    if (!strcmp(argv[1], "giant"))
    {
        bool referenced = false;
        for (int i = 4; i + 1 < argc; ++i)
            if (!strcmp(argv[i], "--exchange")) referenced = !strcmp(argv[i + 1], "referenced");
        return run_giant(argv[2], argv[3], P, std::max(1, arg_int(argc, argv, "--levels", 2)), arg_int(argc, argv, "--chunks", 4), iters, referenced);
    }
    die("the first argument must be shard or giant");
}
