/* CPU oracle of the graph-analytics workloads - TEST INFRASTRUCTURE ONLY, never linked into or
 * called by the product.
 *
 * A sequential restatement of the reference's four algorithms (src/workloads/graphcompute.cu): each
 * function is the host loop of a `compute` method with its kernels run one vertex after another in
 * ascending order, in the reference's data types (64-bit offsets and neighbour ids, 32-bit labels,
 * distances and weights, 64-bit component ids, float ranks).  The reference's kernels race on the
 * arrays they lower, so its iteration counts depend on timing; the results at the fixed point do
 * not, and those are what the parity tests compare (PageRank: within a tolerance, its float sums are
 * order-dependent in the reference too).
 *
 * Pinned by tests/test_graph_oracle_cpu.py against scipy.sparse.csgraph (breadth-first levels,
 * Dijkstra distances, connected components) and a dense power iteration, and on a GPU against the
 * reference's own kernels (oracle/_ref/libgraphcompute_ref.so, tests/test_gpu_graphwl.py). */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GRO_INFINITY 0xFFFFFFFFu /* MYINFINITY, include/workloads/graphcompute.h:14 */

/* BFS::compute (graphcompute.cu:184-202) over bfs_kernel_coalesce (:149-170).  Returns the number
 * of kernel launches (levels + 1). */
int gro_bfs(uint64_t n, const uint64_t *row, const uint64_t *adj, uint32_t src, uint32_t *label) {
    memset(label, 0xFF, n * sizeof(uint32_t));
    label[src] = 0;
    uint32_t level = 0;
    int iter = 0, changed;
    do {
        changed = 0;
        for (uint64_t u = 0; u < n; ++u) {
            if (label[u] != level) continue;
            for (uint64_t i = row[u]; i < row[u + 1]; ++i) {
                const uint64_t next = adj[i];
                if (label[next] == GRO_INFINITY) {
                    label[next] = level + 1;
                    changed = 1;
                }
            }
        }
        ++iter;
        ++level;
    } while (changed);
    return iter;
}

/* CC::compute (graphcompute.cu:108-135) over cc_kernel_coalesce (:57-93). */
int gro_cc(uint64_t n, const uint64_t *row, const uint64_t *adj, unsigned long long *comp) {
    unsigned char *curr = malloc(n ? n : 1), *next = malloc(n ? n : 1);
    for (uint64_t v = 0; v < n; ++v) comp[v] = v;
    memset(curr, 1, n);
    memset(next, 0, n);
    int iter = 0, changed;
    do {
        changed = 0;
        for (uint64_t u = 0; u < n; ++u) {
            if (!curr[u]) continue;
            for (uint64_t i = row[u]; i < row[u + 1]; ++i) {
                const unsigned long long comp_src = comp[u];
                const uint64_t nb = adj[i];
                const unsigned long long comp_next = comp[nb];
                if (comp_next != comp_src) {
                    uint64_t target;
                    unsigned long long value;
                    if (comp_src < comp_next) {
                        target = nb;
                        value = comp_src;
                    } else {
                        target = u;
                        value = comp_next;
                    }
                    if (value < comp[target]) comp[target] = value; /* atomicMin */
                    next[target] = 1;
                    changed = 1;
                }
            }
        }
        memset(curr, 0, n);
        unsigned char *t = curr;
        curr = next;
        next = t;
        ++iter;
    } while (changed);
    free(curr);
    free(next);
    return iter;
}

/* SSSP::compute (graphcompute.cu:357-382) over sssp_kernel_coalesce (:297-318) and sssp_update
 * (:320-330). */
int gro_sssp(uint64_t n, const uint64_t *row, const uint64_t *adj, const uint32_t *weight, uint32_t src,
             uint32_t *cost) {
    uint32_t *new_cost = malloc((n ? n : 1) * sizeof(uint32_t));
    unsigned char *label = calloc(n ? n : 1, 1);
    memset(cost, 0xFF, n * sizeof(uint32_t));
    memset(new_cost, 0xFF, n * sizeof(uint32_t));
    label[src] = 1;
    cost[src] = 0;
    new_cost[src] = 0;
    int iter = 0, changed;
    do {
        changed = 0;
        for (uint64_t u = 0; u < n; ++u) {
            if (!label[u]) continue;
            const uint32_t c = new_cost[u];
            for (uint64_t i = row[u]; i < row[u + 1]; ++i) {
                if (new_cost[u] != c) break;
                if (new_cost[adj[i]] > c + weight[i]) new_cost[adj[i]] = c + weight[i]; /* atomicMin */
            }
            label[u] = 0;
        }
        for (uint64_t v = 0; v < n; ++v)
            if (new_cost[v] < cost[v]) {
                cost[v] = new_cost[v];
                label[v] = 1;
                changed = 1;
            }
        ++iter;
    } while (changed);
    free(new_cost);
    free(label);
    return iter;
}

/* PageRank::compute (graphcompute.cu:267-283) over pr_initialize (:213-221), pr_kernel_coalesce
 * (:223-239) and pr_update (:241-250); alpha, tolerance and max_iter as
 * include/workloads/graphcompute.h:84-86. */
int gro_pagerank(uint64_t n, const uint64_t *row, const uint64_t *adj, float alpha, float tolerance, int max_iter,
                 float *value) {
    float *delta = malloc((n ? n : 1) * sizeof(float)), *residual = malloc((n ? n : 1) * sizeof(float));
    unsigned char *label = malloc(n ? n : 1);
    for (uint64_t v = 0; v < n; ++v) {
        value[v] = 1.0f - alpha;
        delta[v] = (1.0f - alpha) * alpha / (float)(row[v + 1] - row[v]);
        residual[v] = 0.0f;
        label[v] = 1;
    }
    int iter = 0, changed;
    do {
        changed = 0;
        for (uint64_t u = 0; u < n; ++u) {
            if (!label[u]) continue;
            for (uint64_t i = row[u]; i < row[u + 1]; ++i) residual[adj[i]] += delta[u]; /* atomicAdd */
            label[u] = 0;
        }
        for (uint64_t v = 0; v < n; ++v)
            if (residual[v] > tolerance) {
                value[v] += residual[v];
                delta[v] = residual[v] * alpha / (float)(row[v + 1] - row[v]);
                residual[v] = 0.0f;
                label[v] = 1;
                changed = 1;
            }
        ++iter;
    } while (changed && iter < max_iter);
    free(delta);
    free(residual);
    free(label);
    return iter;
}
