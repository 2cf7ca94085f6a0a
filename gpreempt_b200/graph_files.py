"""Graph files for the graph-analytics workloads ("bfs", "sssp", "cc", "pagerank").

The reference reads its graphs in the EMOGI "bel" layout (read_graph, src/workloads/graphcompute.cu:15-45;
weights: SSSP::SSSP, :345-353): three binary files beside one another,

    <prefix>.col   u64 count (= vertices + 1), u64 element type, count x u64 edge offsets
    <prefix>.dst   u64 count (= edges),        u64 element type, count x u64 neighbour ids
    <prefix>.val   u64 count (= edges),        u64 (unused),     count x u32 edge weights

and evaluates on `crankseg_1` of the SuiteSparse collection (config/Z.json:38), a symmetric
structural-mechanics matrix of 52 804 rows and about 10.6 million non-zeros.  That file is not
part of either repository.  This module writes the layout from a matrix the user has
(`--from-mtx`, MatrixMarket through scipy) or from a seeded synthetic graph with the same size
and shape: a symmetric banded graph, every vertex tied to random vertices within a window around
its own index, as a bandwidth-reduced finite-element mesh is.

    python -m gpreempt_b200.graph_files --out /data/crank/crank.bel [--vertices 52804 --degree 201 --band 1500 --seed 1]
    python -m gpreempt_b200.graph_files --out /data/crankseg_1/crankseg_1.bel --from-mtx crankseg_1.mtx
"""
from __future__ import annotations

import argparse
import os

import numpy as np

ELEMENT_TYPE_U64 = 8  # the readers ignore this header word


def write_bel(prefix: str, offsets: np.ndarray, neighbours: np.ndarray, weights: np.ndarray | None = None) -> None:
    offsets = np.ascontiguousarray(offsets, np.uint64)
    neighbours = np.ascontiguousarray(neighbours, np.uint64)
    if offsets[0] != 0 or offsets[-1] != len(neighbours) or np.any(np.diff(offsets.astype(np.int64)) < 0):
        raise ValueError("offsets must start at 0, never decrease and end at the number of edges")
    if len(neighbours) and int(neighbours.max()) >= len(offsets) - 1:
        raise ValueError("a neighbour id is not a vertex")
    os.makedirs(os.path.dirname(os.path.abspath(prefix)), exist_ok=True)
    with open(prefix + ".col", "wb") as f:
        np.array([len(offsets), ELEMENT_TYPE_U64], np.uint64).tofile(f)
        offsets.tofile(f)
    with open(prefix + ".dst", "wb") as f:
        np.array([len(neighbours), ELEMENT_TYPE_U64], np.uint64).tofile(f)
        neighbours.tofile(f)
    if weights is not None:
        weights = np.ascontiguousarray(weights, np.uint32)
        if len(weights) != len(neighbours):
            raise ValueError("one weight per edge")
        with open(prefix + ".val", "wb") as f:
            np.array([len(weights), 4], np.uint64).tofile(f)
            weights.tofile(f)


def read_bel(prefix: str) -> tuple[np.ndarray, np.ndarray, np.ndarray | None]:
    def array(path, dtype):
        with open(path, "rb") as f:
            count = int(np.fromfile(f, np.uint64, 2)[0])
            return np.fromfile(f, dtype, count)

    offsets = array(prefix + ".col", np.uint64)
    neighbours = array(prefix + ".dst", np.uint64)
    weights = array(prefix + ".val", np.uint32) if os.path.exists(prefix + ".val") else None
    return offsets, neighbours, weights


def csr_from_pairs(vertices: int, src: np.ndarray, dst: np.ndarray, symmetric: bool = True):
    """Offsets and sorted neighbour lists of the given edges, without self loops and duplicates."""
    src = np.asarray(src, np.int64)
    dst = np.asarray(dst, np.int64)
    if symmetric:
        src, dst = np.concatenate([src, dst]), np.concatenate([dst, src])
    keep = src != dst
    key = np.unique(src[keep] * vertices + dst[keep])
    s, d = key // vertices, key % vertices
    offsets = np.zeros(vertices + 1, np.uint64)
    np.cumsum(np.bincount(s, minlength=vertices), out=offsets[1:])
    return offsets, d.astype(np.uint64)


def synthetic_banded(vertices: int, degree: int, band: int, seed: int, components: int = 1):
    """A symmetric graph of about `degree` neighbours per vertex, all within `band` of the vertex's
    own index.  With `components` > 1 the index range is cut into that many pieces with no edge
    between them."""
    rng = np.random.default_rng(seed)
    half = max(1, degree // 2)
    src = np.repeat(np.arange(vertices, dtype=np.int64), half)
    off = rng.integers(1, band + 1, size=src.size) * rng.choice(np.array([-1, 1]), size=src.size)
    dst = src + off
    piece = -(-vertices // components)
    ok = (dst >= 0) & (dst < vertices) & (src // piece == dst // piece)
    # a chain through every piece keeps each of them connected
    chain = np.arange(vertices - 1, dtype=np.int64)
    chain = chain[chain // piece == (chain + 1) // piece]
    return csr_from_pairs(vertices, np.concatenate([src[ok], chain]), np.concatenate([dst[ok], chain + 1]))


def synthetic_weights(edges: int, seed: int, high: int = 64) -> np.ndarray:
    return np.random.default_rng(seed + 7919).integers(1, high + 1, size=edges, dtype=np.uint32)


def write_synthetic(prefix: str, vertices: int = 52804, degree: int = 201, band: int = 1500, seed: int = 1,
                    components: int = 1) -> dict:
    offsets, neighbours = synthetic_banded(vertices, degree, band, seed, components)
    write_bel(prefix, offsets, neighbours, synthetic_weights(len(neighbours), seed))
    return {"prefix": prefix, "vertices": vertices, "edges": int(len(neighbours))}


def write_from_mtx(prefix: str, mtx: str, seed: int = 1) -> dict:
    from scipy.io import mmread
    from scipy.sparse import csr_matrix

    m = csr_matrix(mmread(mtx, spmatrix=False))
    m.sort_indices()
    write_bel(prefix, m.indptr, m.indices, synthetic_weights(m.nnz, seed))
    return {"prefix": prefix, "vertices": int(m.shape[0]), "edges": int(m.nnz)}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True, help="prefix of the .col/.dst/.val files")
    ap.add_argument("--from-mtx", default="")
    ap.add_argument("--vertices", type=int, default=52804)
    ap.add_argument("--degree", type=int, default=201)
    ap.add_argument("--band", type=int, default=1500)
    ap.add_argument("--components", type=int, default=1)
    ap.add_argument("--seed", type=int, default=1)
    a = ap.parse_args()
    if a.from_mtx:
        print(write_from_mtx(a.out, a.from_mtx, a.seed))
    else:
        print(write_synthetic(a.out, a.vertices, a.degree, a.band, a.seed, a.components))


if __name__ == "__main__":
    main()
