// Graph-analytics workloads: kernels, graph files and the kernel list of one request (graphwl.h).
#include "graphwl.h"

#include "common.h"
#include "model.h"

#include <algorithm>
#include <cstdlib>
#include <vector>

namespace gpx {

namespace {

__device__ __forceinline__ unsigned warp_min(unsigned v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
    // a fixed tree, so the sum of a vertex does not depend on who ran it or when
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr int kGwUnroll = 8;  // neighbour ids a lane fetches before it follows any of them: 256 edges a round

// Breadth-first search, one level (bfs_kernel_coalesce, graphcompute.cu:149-170): every vertex of
// the current level labels its unlabelled neighbours with the next one.  All writers of a label
// store the same value.
__device__ __forceinline__ void bfs_vertex(const GraphWlParams &p, unsigned u, unsigned long long beg,
                                           unsigned long long end, int lane) {
    const unsigned level = (unsigned)p.iter;
    bool found = false;
    for (unsigned long long i = beg + lane; i < end; i += 32 * kGwUnroll) {
        unsigned v[kGwUnroll], l[kGwUnroll];
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) v[k] = i + 32 * k < end ? p.adj[i + 32 * k] : u;
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) l[k] = p.a[v[k]];
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k)
            if (l[k] == kGwInfinity) {
                p.a[v[k]] = level + 1;
                found = true;
            }
    }
    if (__any_sync(0xffffffffu, found) && lane == 0) p.active[p.iter + 1] = 1;
}

// Shortest paths, relaxation (sssp_kernel_coalesce, graphcompute.cu:297-318): every vertex whose
// distance dropped in the last iteration offers it to its neighbours.  The distance offered is
// cost[u], which only the update pass writes (the reference reads the array that is being lowered).
__device__ __forceinline__ void sssp_vertex(const GraphWlParams &p, unsigned u, unsigned long long beg,
                                            unsigned long long end, int lane) {
    const unsigned cu = p.a[u];
    for (unsigned long long i = beg + lane; i < end; i += 32 * kGwUnroll) {
        unsigned v[kGwUnroll], w[kGwUnroll], c[kGwUnroll];
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) {
            const bool in = i + 32 * k < end;
            v[k] = in ? p.adj[i + 32 * k] : u;
            w[k] = in ? p.wgt[i + 32 * k] : 0u;
        }
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) c[k] = p.b[v[k]];
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) {
            const unsigned nv = cu + w[k];
            if (v[k] != u && c[k] > nv) atomicMin(p.b + v[k], nv);
        }
    }
    __syncwarp();
    if (lane == 0) p.f0[u] = 0;
}

// Connected components, hooking.  The reference (cc_kernel_coalesce, graphcompute.cu:57-93) offers the
// smaller component id along every edge of the vertices that changed and repeats until nothing
// moves, which takes as many launches as the graph is deep when ids are read from a stable copy.
// Here every iteration hooks and then shortcuts (the scheme of Shiloach and Vishkin as in FastSV):
// the smallest id m among u and its neighbours is offered to u and to the vertex u currently names,
// X[u]; the vertex pass then replaces every id by the id that one names.  Ids are read from X and
// offered to Y with atomicMin only, so the outcome of a pass does not depend on the order of its
// warps, and the number of iterations is logarithmic in the depth.  Every id a vertex ever holds is
// a vertex of its own component, ids only fall, and a pass that changes nothing leaves all ends of
// every edge equal: the fixed point is the smallest vertex id of each component, as in the reference.
__device__ __forceinline__ void cc_vertex(const GraphWlParams &p, unsigned u, unsigned long long beg,
                                          unsigned long long end, int lane) {
    const unsigned xu = p.a[u];
    unsigned m = xu;
    for (unsigned long long i = beg + lane; i < end; i += 32 * kGwUnroll) {
        unsigned v[kGwUnroll];
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) v[k] = i + 32 * k < end ? p.adj[i + 32 * k] : u;
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) m = min(m, p.a[v[k]]);
    }
    m = warp_min(m);
    if (lane == 0) {
        atomicMin(p.b + u, m);
        if (m < xu) atomicMin(p.b + xu, m);
    }
}

// PageRank, one iteration (pr_kernel_coalesce + pr_update, graphcompute.cu:223-250) as a gather:
// the residual of v grows by the delta of every in-neighbour (0 for those that did not move last
// time), summed in a fixed order instead of by atomicAdd, and v is updated in the same pass.
__device__ __forceinline__ void pagerank_vertex(const GraphWlParams &p, unsigned v, unsigned long long beg,
                                                unsigned long long end, int lane) {
    const float *dold = reinterpret_cast<const float *>((p.iter & 1) ? p.d1 : p.d0);
    float *dnew = reinterpret_cast<float *>((p.iter & 1) ? p.d0 : p.d1);
    float *value = reinterpret_cast<float *>(p.a), *residual = reinterpret_cast<float *>(p.b);
    // what the update at the end needs, fetched while the edges are walked
    float left = 0.f, val = 0.f, deg = 1.f;
    if (lane == 0) {
        left = residual[v];
        val = value[v];
        deg = (float)p.outdeg[v];
    }
    float s = 0.f;
    for (unsigned long long i = beg + lane; i < end; i += 32 * kGwUnroll) {
        unsigned u[kGwUnroll];
        float d[kGwUnroll];
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) u[k] = i + 32 * k < end ? p.adj[i + 32 * k] : kGwInfinity;
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) d[k] = u[k] != kGwInfinity ? dold[u[k]] : 0.f;
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) s += d[k];
    }
    s = warp_sum(s);
    if (lane == 0) {
        const float r = left + s;
        if (r > p.tol) {
            value[v] = val + r;
            dnew[v] = r * p.alpha / deg;
            residual[v] = 0.f;
            p.active[p.iter + 1] = 1;
        } else {
            residual[v] = r;
            dnew[v] = 0.f;
        }
    }
}

// Two neighbouring vertices at once: their edge lists are walked in the same rounds, so twice as many
// loads are in flight per lane and the pair costs the latency chain of one.  Each vertex's sum is
// taken in the same order as pagerank_vertex takes it, so it does not matter which of the two
// functions a vertex meets.
__device__ __forceinline__ void pagerank_pair(const GraphWlParams &p, unsigned v0, unsigned long long b0,
                                              unsigned long long e0, unsigned long long b1, unsigned long long e1,
                                              int lane) {
    const float *dold = reinterpret_cast<const float *>((p.iter & 1) ? p.d1 : p.d0);
    float *dnew = reinterpret_cast<float *>((p.iter & 1) ? p.d0 : p.d1);
    float *value = reinterpret_cast<float *>(p.a), *residual = reinterpret_cast<float *>(p.b);
    float left = 0.f, val = 0.f, deg = 1.f;  // lane 0: v0, lane 1: v0 + 1
    if (lane < 2) {
        left = residual[v0 + lane];
        val = value[v0 + lane];
        deg = (float)p.outdeg[v0 + lane];
    }
    float s0 = 0.f, s1 = 0.f;
    unsigned long long i0 = b0 + lane, i1 = b1 + lane;
    while (i0 - lane < e0 || i1 - lane < e1) {
        unsigned u0[kGwUnroll], u1[kGwUnroll];
        float d0[kGwUnroll], d1[kGwUnroll];
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) {
            u0[k] = i0 + 32 * k < e0 ? p.adj[i0 + 32 * k] : kGwInfinity;
            u1[k] = i1 + 32 * k < e1 ? p.adj[i1 + 32 * k] : kGwInfinity;
        }
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) {
            d0[k] = u0[k] != kGwInfinity ? dold[u0[k]] : 0.f;
            d1[k] = u1[k] != kGwInfinity ? dold[u1[k]] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < kGwUnroll; ++k) {
            s0 += d0[k];
            s1 += d1[k];
        }
        i0 += 32 * kGwUnroll;
        i1 += 32 * kGwUnroll;
    }
    s0 = warp_sum(s0);
    s1 = warp_sum(s1);
    if (lane < 2) {
        const unsigned v = v0 + lane;
        const float r = left + (lane == 0 ? s0 : s1);
        if (r > p.tol) {
            value[v] = val + r;
            dnew[v] = r * p.alpha / deg;
            residual[v] = 0.f;
            p.active[p.iter + 1] = 1;
        } else {
            residual[v] = r;
            dnew[v] = 0.f;
        }
    }
}

// One tile of an edge pass: p.tile_verts neighbouring vertices, an eighth of them per warp.  The
// first lanes of a warp fetch, for its vertices at once, whether the vertex takes part and where its
// edge list lies; the warp then walks the lists one after another (PageRank: two at a time).  Neighbouring vertices of a
// graph with locality share neighbours, so their reads of labels, distances, ids and deltas hit the
// same cache lines (tiles of vertices spread over the whole graph were tried: 1.8 to 2.7 times slower
// on the searches).
template <int ALGO>
__device__ __forceinline__ void edge_tile(const GraphWlParams &p, int tile) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int per_warp = p.tile_verts / (kGwThreads / 32);
    const unsigned long long first = (unsigned long long)tile * p.tile_verts + wid * per_warp;
    const unsigned long long mine = first + lane;
    bool act = false;
    unsigned long long beg = 0, end = 0;
    if (lane < per_warp && mine < p.n) {
        if (ALGO == GW_BFS) act = p.a[mine] == (unsigned)p.iter;
        if (ALGO == GW_SSSP) act = p.f0[mine] != 0;
        if (ALGO == GW_CC || ALGO == GW_PAGERANK) act = true;
        if (act) {
            beg = p.row[mine];
            end = p.row[mine + 1];
        }
    }
    if (ALGO == GW_PAGERANK) {
        // every vertex takes part: walk the lists two at a time
        int j = 0;
#pragma unroll 1
        for (; j + 1 < per_warp && first + j + 1 < p.n; j += 2)
            pagerank_pair(p, (unsigned)(first + j), __shfl_sync(0xffffffffu, beg, j), __shfl_sync(0xffffffffu, end, j),
                          __shfl_sync(0xffffffffu, beg, j + 1), __shfl_sync(0xffffffffu, end, j + 1), lane);
        if (j < per_warp && first + j < p.n)
            pagerank_vertex(p, (unsigned)(first + j), __shfl_sync(0xffffffffu, beg, j), __shfl_sync(0xffffffffu, end, j), lane);
        return;
    }
#pragma unroll 1
    for (int j = 0; j < per_warp; ++j) {
        if (!__shfl_sync(0xffffffffu, act ? 1 : 0, j)) continue;
        const unsigned long long b = __shfl_sync(0xffffffffu, beg, j), e = __shfl_sync(0xffffffffu, end, j);
        const unsigned u = (unsigned)(first + j);
        if (ALGO == GW_BFS) bfs_vertex(p, u, b, e, lane);
        if (ALGO == GW_SSSP) sssp_vertex(p, u, b, e, lane);
        if (ALGO == GW_CC) cc_vertex(p, u, b, e, lane);
    }
}

// sssp_update (graphcompute.cu:320-330): a vertex whose offered distance is below its own takes it and
// is in the next frontier.  Components: the shortcut, X[v] = min(Y[v], Y[Y[v]]).
template <int ALGO>
__device__ __forceinline__ bool vertex_tile(const GraphWlParams &p, int tile) {
    bool found = false;
    for (int k = 0; k < kGwVertexTileVerts / kGwThreads; ++k) {
        const unsigned long long v = (unsigned long long)tile * kGwVertexTileVerts + k * kGwThreads + threadIdx.x;
        if (v >= p.n) break;
        if (ALGO == GW_SSSP) {
            const unsigned nb = p.b[v];
            if (nb < p.a[v]) {
                p.a[v] = nb;
                p.f0[v] = 1;
                found = true;
            }
        } else {
            const unsigned y = p.b[v];
            const unsigned nw = min(y, p.b[y]);
            if (nw < p.a[v]) {
                p.a[v] = nw;
                found = true;
            }
        }
    }
    return found;
}

// What CC::compute, BFS::compute, pr_initialize and SSSP::compute set up before their loops
// (graphcompute.cu:109-114, 188-189, 213-221, 361-366), plus the iteration flags.
__device__ __forceinline__ void init_tile(const GraphWlParams &p, int tile) {
    if (tile == 0) {
        for (int i = threadIdx.x; i <= kGwMaxIters; i += kGwThreads) p.active[i] = i == 0 ? 1 : 0;
    }
    for (int k = 0; k < kGwVertexTileVerts / kGwThreads; ++k) {
        const unsigned long long vv = (unsigned long long)tile * kGwVertexTileVerts + k * kGwThreads + threadIdx.x;
        if (vv >= p.n) break;
        const unsigned v = (unsigned)vv;
        if (p.algo == GW_BFS) {
            p.a[v] = v == p.src ? 0u : kGwInfinity;
        } else if (p.algo == GW_SSSP) {
            p.a[v] = p.b[v] = v == p.src ? 0u : kGwInfinity;
            p.f0[v] = v == p.src ? 1 : 0;
        } else if (p.algo == GW_CC) {
            p.a[v] = p.b[v] = v;
        } else {
            reinterpret_cast<float *>(p.a)[v] = 1.0f - p.alpha;
            reinterpret_cast<float *>(p.b)[v] = 0.0f;
            reinterpret_cast<float *>(p.d0)[v] = (1.0f - p.alpha) * p.alpha / (float)p.outdeg[v];
            reinterpret_cast<float *>(p.d1)[v] = 0.0f;
        }
    }
}

template <int ALGO, int PHASE>
__global__ void __launch_bounds__(kGwThreads)
graphwl_kernel(const __grid_constant__ GraphWlParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (PHASE != GW_INIT && p.active[p.iter] == 0) {
        // No flag for this iteration.  With the preempt word down that is final: every kernel before
        // this one ran to its end (the word stays up from the moment a kernel stops until the stream
        // is idle), so this one is behind the last live iteration, has nothing to do, and its tiles
        // count as run.  With the word up a predecessor may have stopped before it raised the flag:
        // the kernel then goes on to the claim below, which records it as a stop point, and it is
        // judged again when the run is resumed.
        if (dynamic) {
            if (threadIdx.x == 0) s_tile = load_word(blp.preempted);
            __syncthreads();
        }
        if (!dynamic || s_tile == 0) {
            if (blockIdx.x == 0 && threadIdx.x == 0) {
                int had = 0;
                if (dynamic) had = atomicMax(blp.executed, blp.total_tiles);
                if (blp.trace && had < blp.total_tiles) {
                    const unsigned long long t = globaltimer_ns();
                    atomicMin(blp.trace + 0, t);
                    atomicMax(blp.trace + 1, t);
                    atomicAdd(blp.trace + 3, (unsigned long long)(blp.total_tiles - had));
                }
            }
            return;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) trace_begin(blp);
    int iter = 0;
    bool found = false;
    for (;;) {
        int tile;
        if (dynamic) {
            if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
            __syncthreads();
            tile = s_tile;
        } else {
            tile = blp_claim(blp, iter);
        }
        if (tile < 0) break;
        if (PHASE == GW_INIT) init_tile(p, tile);
        if (PHASE == GW_EDGES) edge_tile<ALGO>(p, tile);
        if (PHASE == GW_VERTICES) found |= vertex_tile<ALGO>(p, tile);
        ++iter;
        if (dynamic) __syncthreads();
    }
    if (PHASE == GW_VERTICES) {
        if (__syncthreads_or(found ? 1 : 0) && threadIdx.x == 0) p.active[p.iter + 1] = 1;
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

typedef void (*GraphKernel)(const GraphWlParams, BlpArgs);

GraphKernel pick_kernel(const GraphWlParams &p) {
    if (p.phase == GW_INIT) return graphwl_kernel<GW_BFS, GW_INIT>;
    if (p.phase == GW_VERTICES) return p.algo == GW_SSSP ? graphwl_kernel<GW_SSSP, GW_VERTICES> : graphwl_kernel<GW_CC, GW_VERTICES>;
    switch (p.algo) {
        case GW_BFS: return graphwl_kernel<GW_BFS, GW_EDGES>;
        case GW_SSSP: return graphwl_kernel<GW_SSSP, GW_EDGES>;
        case GW_CC: return graphwl_kernel<GW_CC, GW_EDGES>;
        default: return graphwl_kernel<GW_PAGERANK, GW_EDGES>;
    }
}

// ---- graph files ---------------------------------------------------------------------------------

struct HostGraph {
    uint64_t n = 0, e = 0;
    std::vector<unsigned long long> row;
    std::vector<unsigned> adj, wgt;
};

struct File {
    FILE *fp = nullptr;
    ~File() {
        if (fp) fclose(fp);
    }
};

// One array file of the layout read_graph reads (graphcompute.cu:15-45): u64 element count, u64
// element type (ignored there and here), then the elements.
template <typename T>
int read_array(const std::string &path, std::vector<T> &out) {
    File f;
    f.fp = fopen(path.c_str(), "rb");
    GPX_REQUIRE(f.fp, GPX_NOT_FOUND, "graph file '%s' cannot be opened", path.c_str());
    uint64_t head[2] = {0, 0};
    GPX_REQUIRE(fread(head, sizeof(uint64_t), 2, f.fp) == 2, GPX_FAIL, "graph file '%s' has no header", path.c_str());
    GPX_REQUIRE(head[0] < (1ull << 36), GPX_OUT_OF_RANGE, "graph file '%s' claims %llu elements", path.c_str(),
                (unsigned long long)head[0]);
    out.resize(head[0]);
    GPX_REQUIRE(fread(out.data(), sizeof(T), out.size(), f.fp) == out.size(), GPX_FAIL,
                "graph file '%s' is shorter than its header says (%llu elements)", path.c_str(),
                (unsigned long long)head[0]);
    return GPX_SUCC;
}

int read_graph_files(const std::string &prefix, bool weights, HostGraph &g) {
    std::vector<unsigned long long> dst;
    GPX_TRY(read_array(prefix + ".col", g.row));
    GPX_TRY(read_array(prefix + ".dst", dst));
    GPX_REQUIRE(g.row.size() >= 2, GPX_FAIL, "graph '%s' has no vertices", prefix.c_str());
    g.n = g.row.size() - 1;
    g.e = dst.size();
    GPX_REQUIRE(g.n < kGwInfinity, GPX_OUT_OF_RANGE, "graph '%s': %llu vertices, at most 2^32 - 2 are supported",
                prefix.c_str(), (unsigned long long)g.n);
    GPX_REQUIRE(g.row[0] == 0 && g.row[g.n] == g.e, GPX_FAIL,
                "graph '%s': offsets run from %llu to %llu but there are %llu edges", prefix.c_str(),
                (unsigned long long)g.row[0], (unsigned long long)g.row[g.n], (unsigned long long)g.e);
    for (uint64_t v = 0; v < g.n; ++v)
        GPX_REQUIRE(g.row[v] <= g.row[v + 1], GPX_FAIL, "graph '%s': offsets decrease at vertex %llu", prefix.c_str(),
                    (unsigned long long)v);
    g.adj.resize(g.e);
    for (uint64_t i = 0; i < g.e; ++i) {
        GPX_REQUIRE(dst[i] < g.n, GPX_FAIL, "graph '%s': edge %llu points at vertex %llu of %llu", prefix.c_str(),
                    (unsigned long long)i, (unsigned long long)dst[i], (unsigned long long)g.n);
        g.adj[i] = (unsigned)dst[i];
    }
    if (weights) {
        // SSSP::SSSP, graphcompute.cu:345-353: 32-bit weights, one per edge.
        GPX_TRY(read_array(prefix + ".val", g.wgt));
        GPX_REQUIRE(g.wgt.size() >= g.e, GPX_FAIL, "graph '%s': %zu weights for %llu edges", prefix.c_str(),
                    g.wgt.size(), (unsigned long long)g.e);
        g.wgt.resize(g.e);
    }
    return GPX_SUCC;
}

// In-edge lists, sources in ascending order.
void transpose(const HostGraph &g, std::vector<unsigned long long> &trow, std::vector<unsigned> &tadj) {
    trow.assign(g.n + 1, 0);
    for (uint64_t i = 0; i < g.e; ++i) ++trow[g.adj[i] + 1];
    for (uint64_t v = 0; v < g.n; ++v) trow[v + 1] += trow[v];
    tadj.resize(g.e);
    std::vector<unsigned long long> at(trow.begin(), trow.end() - 1);
    for (uint64_t u = 0; u < g.n; ++u)
        for (unsigned long long i = g.row[u]; i < g.row[u + 1]; ++i) tadj[at[g.adj[i]]++] = (unsigned)u;
}

template <typename T>
int to_device(gpx_model &m, const std::vector<T> &host, T **out) {
    T *d = nullptr;
    GPX_CUDA(cudaMalloc((void **)&d, std::max<size_t>(host.size(), 1) * sizeof(T)));
    m.scratch.push_back(d);
    if (!host.empty()) GPX_CUDA(cudaMemcpy(d, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice));
    *out = d;
    return GPX_SUCC;
}

template <typename T>
int device_zeroed(gpx_model &m, size_t n, T **out) {
    T *d = nullptr;
    GPX_CUDA(cudaMalloc((void **)&d, std::max<size_t>(n, 1) * sizeof(T)));
    m.scratch.push_back(d);
    GPX_CUDA(cudaMemset(d, 0, std::max<size_t>(n, 1) * sizeof(T)));
    *out = d;
    return GPX_SUCC;
}

int add_result(gpx_model &m, const char *name, const char *stype, size_t n, unsigned **out) {
    Storage s;
    s.name = name;
    s.stype = stype;
    s.kind = Storage::Vec;
    s.rank = 1;
    s.dims[0] = (int64_t)n;
    s.dims[1] = s.dims[2] = s.dims[3] = 1;
    s.bytes = n * 4;
    GPX_CUDA(cudaMalloc((void **)&s.dptr, std::max<size_t>(s.bytes, 4)));
    GPX_CUDA(cudaMemset(s.dptr, 0, std::max<size_t>(s.bytes, 4)));
    *out = reinterpret_cast<unsigned *>(s.dptr);
    m.add_storage(s);
    return GPX_SUCC;
}

const char *kAlgoNames[4] = {"bfs", "sssp", "cc", "pagerank"};

bool split_name(const std::string &name, int &algo, std::string &path) {
    const size_t colon = name.find(':');
    const std::string head = colon == std::string::npos ? name : name.substr(0, colon);
    for (int a = 0; a < 4; ++a)
        if (head == kAlgoNames[a]) {
            algo = a;
            path = colon == std::string::npos ? std::string() : name.substr(colon + 1);
            return true;
        }
    return false;
}

}  // namespace

int graphwl_grid(const GraphWlParams &p, int total_tiles, int sm_count) {
    int blocks = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, pick_kernel(p), kGwThreads, 0);
    if (blocks < 1) blocks = 1;
    long long grid = (long long)blocks * sm_count;
    if (grid > total_tiles) grid = total_tiles;
    return grid < 1 ? 1 : (int)grid;
}

cudaError_t graphwl_launch(const GraphWlParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    launch_layer(pick_kernel(p), grid, kGwThreads, 0, s, p, blp);
    return cudaGetLastError();
}

bool is_graph_workload(const std::string &name) {
    int algo;
    std::string path;
    return split_name(name, algo, path);
}

int build_graph_workload(gpx_model &m, const std::string &name, const gpx_model_opts &) {
    int algo = 0;
    std::string path;
    GPX_REQUIRE(split_name(name, algo, path), GPX_NOT_FOUND, "unknown model '%s'", name.c_str());
    GPX_REQUIRE(!path.empty(), GPX_NOT_FOUND,
                "'%s' needs a graph: open it as '%s:<prefix of the .col/.dst files>' (client key graph_path)",
                name.c_str(), name.c_str());
    // The reference prepends a directory fixed at build time (GRAPH_BASE_PATH, src/executor.cpp:12);
    // here it comes from the environment.
    if (path[0] != '/') {
        const char *base = getenv("GPX_GRAPH_BASE_PATH");
        if (base && base[0]) path = std::string(base) + "/" + path;
    }
    // The files first: what is wrong with them can be told without a GPU.
    HostGraph g;
    GPX_TRY(read_graph_files(path, algo == GW_SSSP, g));
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    m.device = d.device;
    m.sm_count = d.sm_count;
    m.sci = true;
    m.graph_algo = algo;
    m.graph_vertices = g.n;
    m.graph_edges = g.e;

    GraphWlParams base{};
    base.algo = algo;
    base.n = (unsigned)g.n;
    base.src = 0;
    base.alpha = 0.85f;
    base.tol = 0.001f;
    // Vertices per tile of the edge passes.  The searches touch few vertices per pass, and what a
    // CTA pays per tile is the latency of asking which: larger tiles, fewer rounds.  PageRank walks
    // every edge list in every pass and balances better in small tiles: two vertices per warp, walked
    // together.  (52 804 vertices with about 200 edges each: bfs 1.21 / 0.58 / 0.40 ms a run with 8 /
    // 32 / 64; pagerank, one list at a time, 1.60 / 2.08 / 2.09.)
    {
        const int by_algo[4] = {64, 32, 32, 16};
        base.tile_verts = by_algo[algo];
        const char *e = getenv("GPX_GRAPH_TILE");
        if (e && atoi(e) >= 8) base.tile_verts = std::min(atoi(e) / 8 * 8, kGwEdgeTileVertsMax);
    }
    unsigned long long *row = nullptr;
    unsigned *adj = nullptr;
    if (algo == GW_PAGERANK) {
        std::vector<unsigned long long> trow;
        std::vector<unsigned> tadj, outdeg(g.n);
        transpose(g, trow, tadj);
        for (uint64_t v = 0; v < g.n; ++v) outdeg[v] = (unsigned)(g.row[v + 1] - g.row[v]);
        GPX_TRY(to_device(m, trow, &row));
        GPX_TRY(to_device(m, tadj, &adj));
        unsigned *deg = nullptr;
        GPX_TRY(to_device(m, outdeg, &deg));
        base.outdeg = deg;
    } else {
        GPX_TRY(to_device(m, g.row, &row));
        GPX_TRY(to_device(m, g.adj, &adj));
    }
    base.row = row;
    base.adj = adj;
    if (algo == GW_SSSP) {
        unsigned *w = nullptr;
        GPX_TRY(to_device(m, g.wgt, &w));
        base.wgt = w;
    }
    const char *result[4] = {"label", "cost", "comp", "value"};
    GPX_TRY(add_result(m, result[algo], algo == GW_PAGERANK ? "float32" : "uint32", g.n, &base.a));
    if (algo != GW_BFS) GPX_TRY(device_zeroed(m, g.n, &base.b));
    if (algo == GW_PAGERANK) {
        GPX_TRY(device_zeroed(m, g.n, &base.d0));
        GPX_TRY(device_zeroed(m, g.n, &base.d1));
    }
    if (algo == GW_SSSP) GPX_TRY(device_zeroed(m, g.n, &base.f0));
    GPX_TRY(device_zeroed(m, (size_t)kGwMaxIters + 1, &base.active));
    m.graph_active = base.active;

    const int edge_tiles = (int)((g.n + base.tile_verts - 1) / base.tile_verts);
    const int vertex_tiles = (int)((g.n + kGwVertexTileVerts - 1) / kGwVertexTileVerts);
    auto make = [&](int phase, int iter) {
        Kernel k;
        k.type = KernelType::GraphWl;
        GraphWlParams p = base;
        p.phase = phase;
        p.iter = iter;
        k.graphwl = p;
        k.threads = kGwThreads;
        k.total_tiles = phase == GW_EDGES ? edge_tiles : vertex_tiles;
        k.grid = graphwl_grid(p, k.total_tiles, m.sm_count);
        const char *what = phase == GW_INIT ? "init" : (phase == GW_EDGES ? "edges" : "vertices");
        k.name = std::string("graphwl_kernel.") + kAlgoNames[algo] + "." + what +
                 (phase == GW_INIT ? std::string() : "." + std::to_string(iter));
        // per launch: the result array; an edge pass also walks (on average) its share of the edges
        k.bytes = (double)g.n * 8.0;
        k.flops = 0;
        return k;
    };

    // The kernel list: run the algorithm once, iteration by iteration, to see how many it takes.
    // The iterations are race-free, so every later run takes the same number; two more are listed
    // (they return at once) and a run that would need more leaves its last flag up, which
    // gpx_model_graph_info reports as "not converged".  PageRank stops after 100 iterations whatever
    // happens (max_iter, graphcompute.cu:281).
    const int iter_cap = algo == GW_PAGERANK ? 100 : kGwMaxIters - 2;
    BlpArgs plain{};
    cudaStream_t s = nullptr;
    m.kernels.push_back(make(GW_INIT, 0));
    plain.total_tiles = m.kernels.back().total_tiles;
    GPX_CUDA(graphwl_launch(m.kernels.back().graphwl, m.kernels.back().grid, plain, s));
    int live = 0;
    for (int it = 0; it < iter_cap; ++it) {
        int flag = 0;
        GPX_CUDA(cudaMemcpy(&flag, base.active + it, sizeof(int), cudaMemcpyDeviceToHost));
        if (!flag) break;
        ++live;
        const size_t first = m.kernels.size();
        m.kernels.push_back(make(GW_EDGES, it));
        if (algo == GW_SSSP || algo == GW_CC) m.kernels.push_back(make(GW_VERTICES, it));
        for (size_t k = first; k < m.kernels.size(); ++k) {
            plain.total_tiles = m.kernels[k].total_tiles;
            GPX_CUDA(graphwl_launch(m.kernels[k].graphwl, m.kernels[k].grid, plain, s));
        }
    }
    GPX_CUDA(cudaStreamSynchronize(s));
    GPX_REQUIRE(live < kGwMaxIters - 2, GPX_OUT_OF_RANGE, "%s: no fixed point within %d iterations", name.c_str(),
                kGwMaxIters - 2);
    for (int extra = 0; extra < 2 && live + extra < iter_cap; ++extra) {
        m.kernels.push_back(make(GW_EDGES, live + extra));
        if (algo == GW_SSSP || algo == GW_CC) m.kernels.push_back(make(GW_VERTICES, live + extra));
    }
    m.graph_iterations = live;
    // Edge traffic of a whole run, spread over the live edge passes for the per-kernel figures.
    double edge_bytes = (double)g.e * (algo == GW_SSSP ? 12.0 : 8.0);
    if (algo == GW_PAGERANK || algo == GW_CC) edge_bytes = (double)g.e * 4.0 * std::max(live, 1);
    for (Kernel &k : m.kernels)
        if (k.graphwl.phase == GW_EDGES && k.graphwl.iter < live) k.bytes += edge_bytes / std::max(live, 1);
    return GPX_SUCC;
}

}  // namespace gpx

extern "C" {

int gpx_model_graph_info(gpx_model *m, uint64_t *vertices, uint64_t *edges, int *listed_iterations,
                         int *live_iterations, int *converged) {
    using namespace gpx;
    GPX_REQUIRE(m, GPX_FAIL, "NULL model");
    GPX_REQUIRE(m->graph_algo >= 0, GPX_NOT_FOUND, "model '%s' is not a graph workload", m->name.c_str());
    if (vertices) *vertices = m->graph_vertices;
    if (edges) *edges = m->graph_edges;
    int listed = 0;
    for (const Kernel &k : m->kernels)
        if (k.graphwl.phase == GW_EDGES) ++listed;
    if (listed_iterations) *listed_iterations = listed;
    if (live_iterations || converged) {
        std::vector<int> flags((size_t)listed + 1);
        GPX_CUDA(cudaMemcpy(flags.data(), m->graph_active, flags.size() * sizeof(int), cudaMemcpyDeviceToHost));
        int live = 0;
        while (live < listed && flags[live]) ++live;
        if (live_iterations) *live_iterations = live;
        // PageRank may end at its iteration limit with work left, as in the reference.
        if (converged) *converged = flags[listed] == 0 || m->graph_algo == GW_PAGERANK ? 1 : 0;
    }
    return GPX_SUCC;
}

}  // extern "C"
