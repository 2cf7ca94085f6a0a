// miniWeather on the executor's kernel list: twelve preemptible semi-discrete steps per time step.
// Follows src/workloads/miniweather.cu of the reference (initial state :395-507, time step
// :182-200, kernels :222-372, reductions :650-677); arithmetic keeps the reference's types - the
// horizontal flux evaluates density, winds, temperature and pressure in double, everything else
// is float - so that results agree with it to rounding.
#include "stencil.h"

#include "model.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <thread>
#include <vector>

namespace gpx {

namespace {

// Physical constants of the reference (miniweather.cu:35-52), `real` = float.
constexpr float kPi = 3.14159265358979323846264338327;
constexpr float kGrav = 9.8;
constexpr float kCp = 1004.;
constexpr float kCv = 717.;
constexpr float kRd = 287.;
constexpr float kP0 = 1.e5;
constexpr float kC0 = 27.5629410929725921310572974482;
constexpr float kGamm = 1.40027894002789400278940027894;
constexpr float kXlen = 2.e4;
constexpr float kZlen = 1.e4;
constexpr float kHvBeta = 0.05;
constexpr float kCfl = 1.50;
constexpr float kMaxSpeed = 450;
constexpr int ID_DENS = 0, ID_UMOM = 1, ID_WMOM = 2, ID_RHOT = 3;

struct Grid {
    int nx, nz, W;   // W: row stride (nx + 4)
    unsigned plane;  // (nz + 4) * W; four planes stay below 2^31 elements (checked when the model is built)
};

__device__ __forceinline__ Grid grid_of(const StencilParams &p) {
    Grid g;
    g.nx = p.nx;
    g.nz = p.nz;
    g.W = p.nx + 2 * kMwHalo;
    g.plane = (unsigned)(p.nz + 2 * kMwHalo) * (unsigned)g.W;
    return g;
}


// Arithmetic with every rounding written out.  The reference is compiled with nvcc's default
// -fmad=true, which leaves the choice between a fused multiply-add and a rounded product plus a
// sum to the assembler; its choice depends on the surrounding code, so relying on it here would
// tie the results to register pressure.  These are the operations the reference's kernels
// execute (checked on a GPU against that code: all cells of all variables identical).
__device__ __forceinline__ float interp4(float s0, float s1, float s2, float s3) {
    // (-s0 + 7*(s1 + s2) - s3) / 12
    return __fdiv_rn(__fsub_rn(__fmaf_rn(7.f, __fadd_rn(s1, s2), -s0), s3), 12.f);
}
__device__ __forceinline__ float third_derivative(float s0, float s1, float s2, float s3, float hv_coef) {
    // (-s0 + 3*(s1 - s2) + s3) * hv_coef
    return __fmul_rn(__fadd_rn(__fmaf_rn(3.f, __fsub_rn(s1, s2), -s0), s3), hv_coef);
}
__device__ __forceinline__ float advance(float init, float dt, float tend) { return __fmaf_rn(dt, tend, init); }

// Horizontal tile: cells [i0, i1) of row k.  compute_tendencies_x (:222-258) then
// compute_tendencies_x_r (:260-272).  The row segment with two cells on either side is staged in
// shared memory; the cells beyond the ends of the row wrap around as set_halo_values_x (:331-341)
// would have written them, and the tiles at the ends of the row store those halo cells.
__device__ __forceinline__ void tile_x(const StencilParams &p, const Grid &g, int tile, float *smem) {
    constexpr int ldi = kMwTileXMax + 2 * kMwHalo;  // staged values per variable
    constexpr int ldf = kMwTileXMax + 1;            // fluxes per variable
    float *sin = smem, *sflux = smem + kMwVars * ldi;
    const int k = tile / p.tiles_per_row;
    const int i0 = (tile - k * p.tiles_per_row) * p.tile_x;
    const int i1 = min(i0 + p.tile_x, g.nx);
    const int n = i1 - i0;
    const unsigned row = (unsigned)(k + kMwHalo) * (unsigned)g.W;
    const float *__restrict__ forcing = p.forcing;
    // Every global load of the tile is issued up front: the row segment to stage (up to three
    // values per variable and thread) and the cells' starting values, which are not needed until
    // the update and so overlap the flux arithmetic.
    constexpr int kStageIters = (kMwTileXMax + 2 * kMwHalo + kMwThreads - 1) / kMwThreads;
    constexpr int kCellIters = kMwTileXMax / kMwThreads;
    float staged[kStageIters][kMwVars], init_v[kCellIters][kMwVars];
#pragma unroll
    for (int it = 0; it < kStageIters; ++it) {
        const int c = threadIdx.x + it * kMwThreads;
        const int ca = i0 + c;  // array column
        const int src = ca < kMwHalo ? ca + g.nx : (ca >= g.nx + kMwHalo ? ca - g.nx : ca);
#pragma unroll
        for (int ll = 0; ll < kMwVars; ++ll)
            staged[it][ll] = c < n + 2 * kMwHalo ? forcing[ll * g.plane + row + src] : 0.f;
    }
#pragma unroll
    for (int it = 0; it < kCellIters; ++it) {
        const int f = threadIdx.x + it * kMwThreads;
#pragma unroll
        for (int ll = 0; ll < kMwVars; ++ll)
            init_v[it][ll] = f < n ? p.init[ll * g.plane + row + (unsigned)(i0 + f + kMwHalo)] : 0.f;
    }
#pragma unroll
    for (int it = 0; it < kStageIters; ++it) {
        const int c = threadIdx.x + it * kMwThreads;
        const int ca = i0 + c;
        if (c < n + 2 * kMwHalo) {
            const bool halo = ca < kMwHalo || ca >= g.nx + kMwHalo;
#pragma unroll
            for (int ll = 0; ll < kMwVars; ++ll) {
                sin[ll * ldi + c] = staged[it][ll];
                if (halo) p.forcing[ll * g.plane + row + ca] = staged[it][ll];
            }
        }
    }
    __syncthreads();
    const float hv_coef = __fdiv_rn(__fmul_rn(-kHvBeta, p.dx), __fmul_rn(16.f, p.dt));
    const float hd = p.hy_dens_cell[k + kMwHalo], hdt = p.hy_dens_theta_cell[k + kMwHalo];
    for (int f = threadIdx.x; f <= n; f += kMwThreads) {  // interface between cells i0+f-1 and i0+f
        float vals[kMwVars], d3_vals[kMwVars];
#pragma unroll
        for (int ll = 0; ll < kMwVars; ++ll) {
            const float s0 = sin[ll * ldi + f], s1 = sin[ll * ldi + f + 1];
            const float s2 = sin[ll * ldi + f + 2], s3 = sin[ll * ldi + f + 3];
            vals[ll] = interp4(s0, s1, s2, s3);
            d3_vals[ll] = third_derivative(s0, s1, s2, s3, hv_coef);
        }
        const double r = (double)__fadd_rn(vals[ID_DENS], hd);
        const double u = __ddiv_rn((double)vals[ID_UMOM], r);
        const double w = __ddiv_rn((double)vals[ID_WMOM], r);
        const double t = __ddiv_rn((double)__fadd_rn(vals[ID_RHOT], hdt), r);
        const double pr = __dmul_rn((double)kC0, pow(__dmul_rn(r, t), (double)kGamm));
        const double ru = __dmul_rn(r, u);
        // r*u feeds four fluxes; the mass flux subtracts from the rounded product, the others fuse
        sflux[ID_DENS * ldf + f] = (float)__dsub_rn(ru, (double)d3_vals[ID_DENS]);
        sflux[ID_UMOM * ldf + f] = (float)__dsub_rn(__fma_rn(ru, u, pr), (double)d3_vals[ID_UMOM]);
        sflux[ID_WMOM * ldf + f] = (float)__fma_rn(ru, w, -(double)d3_vals[ID_WMOM]);
        sflux[ID_RHOT * ldf + f] = (float)__fma_rn(ru, t, -(double)d3_vals[ID_RHOT]);
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < kCellIters; ++it) {
        const int f = threadIdx.x + it * kMwThreads;
        if (f < n) {
            const unsigned at = row + (unsigned)(i0 + f + kMwHalo);
#pragma unroll
            for (int ll = 0; ll < kMwVars; ++ll) {
                const float tend = __fdiv_rn(-__fsub_rn(sflux[ll * ldf + f + 1], sflux[ll * ldf + f]), p.dx);
                p.out[ll * g.plane + at] = advance(init_v[it][ll], p.dt, tend);
            }
        }
    }
}

// Value of variable ll in array row ka (a row outside the interior) of column ca as the
// reference's flux kernel reads it after set_halo_values_z (:346-372): the boundary row's value
// (scaled by the density ratio for the horizontal momentum, zero for the vertical momentum) where
// the reference's launch covers the cell, else what the array holds.  A derived value is stored.
__device__ __forceinline__ float halo_row_value(const StencilParams &p, const Grid &g, int ll, int ka, int ca) {
    const unsigned at = ll * g.plane + (unsigned)ka * (unsigned)g.W + (unsigned)ca;
    if (ll * g.W + ca >= p.halo_z_ids) return p.forcing[at];
    float v = 0.f;
    if (ll != ID_WMOM) {
        const bool low = ka < kMwHalo;
        v = p.forcing[ll * g.plane + (unsigned)(low ? kMwHalo : g.nz + kMwHalo - 1) * (unsigned)g.W + (unsigned)ca];
        if (ll == ID_UMOM) v = v * p.halo_ratio[low ? ka : ka - g.nz];
    }
    p.forcing[at] = v;
    return v;
}

// Vertical tile: kMwThreads columns x up to kMwTileZRows rows; one thread walks down one column
// with the four stencil rows of every variable in registers.  compute_tendencies_z (:278-318)
// then compute_tendencies_z_r (:320-336).
__device__ __forceinline__ void tile_z(const StencilParams &p, const Grid &g, int tile) {
    const int tr = tile / p.tiles_cols;
    const int i = (tile - tr * p.tiles_cols) * kMwThreads + (int)threadIdx.x;  // cell column
    if (i >= g.nx) return;
    const int k0 = tr * p.tile_rows;
    const int nr = min(p.tile_rows, g.nz - k0);
    const int ca = i + kMwHalo;
    const float hv_coef = __fdiv_rn(__fmul_rn(-kHvBeta, p.dz), __fmul_rn(16.f, p.dt));
    const float *__restrict__ forcing = p.forcing;
    float win[kMwVars][4];  // array rows k .. k+3 of interface k
#pragma unroll
    for (int ll = 0; ll < kMwVars; ++ll)
#pragma unroll
        for (int s = 0; s < 3; ++s) {
            const int ka = k0 + s;
            win[ll][s + 1] = ka >= kMwHalo ? forcing[ll * g.plane + (unsigned)ka * (unsigned)g.W + (unsigned)ca]
                                           : halo_row_value(p, g, ll, ka, ca);
        }
    // Values of the next step are loaded one step ahead, before this step's stores (out may be
    // the array init points to, so a load could not move above a store by itself).
    float next_row[kMwVars], next_init[kMwVars];
#pragma unroll
    for (int ll = 0; ll < kMwVars; ++ll) {
        const int ka = k0 + 3;
        next_row[ll] = ka < g.nz + kMwHalo ? forcing[ll * g.plane + (unsigned)ka * (unsigned)g.W + (unsigned)ca]
                                           : halo_row_value(p, g, ll, ka, ca);
        next_init[ll] = 0.f;
    }
    float below[kMwVars] = {0.f, 0.f, 0.f, 0.f};  // flux through the interface under the cell about to be updated
    for (int j = 0; j <= nr; ++j) {
        const int k = k0 + j;  // interface below cell row k
        float vals[kMwVars], d3_vals[kMwVars], init_v[kMwVars];
        const unsigned cell = (unsigned)(k - 1 + kMwHalo) * (unsigned)g.W + (unsigned)ca;  // cell above interface k-1
#pragma unroll
        for (int ll = 0; ll < kMwVars; ++ll) {
            win[ll][0] = win[ll][1];
            win[ll][1] = win[ll][2];
            win[ll][2] = win[ll][3];
            win[ll][3] = next_row[ll];
            init_v[ll] = next_init[ll];
        }
        if (j < nr) {
            const int ka = k + 4;  // last row of the next interface's stencil
#pragma unroll
            for (int ll = 0; ll < kMwVars; ++ll) {
                next_row[ll] = ka < g.nz + kMwHalo ? forcing[ll * g.plane + (unsigned)ka * (unsigned)g.W + (unsigned)ca]
                                                   : halo_row_value(p, g, ll, ka, ca);
                next_init[ll] = p.init[ll * g.plane + cell + (unsigned)g.W];  // cell row k, updated next step
            }
        }
#pragma unroll
        for (int ll = 0; ll < kMwVars; ++ll) {
            vals[ll] = interp4(win[ll][0], win[ll][1], win[ll][2], win[ll][3]);
            d3_vals[ll] = third_derivative(win[ll][0], win[ll][1], win[ll][2], win[ll][3], hv_coef);
        }
        const float r = __fadd_rn(vals[ID_DENS], p.hy_dens_int[k]);
        const float u = __fdiv_rn(vals[ID_UMOM], r);
        float w = __fdiv_rn(vals[ID_WMOM], r);
        const float t = __fdiv_rn(__fadd_rn(vals[ID_RHOT], p.hy_dens_theta_int[k]), r);
        const float pr = __fmaf_rn(kC0, powf(__fmul_rn(r, t), kGamm), -p.hy_pressure_int[k]);
        if (k == 0 || k == g.nz) {
            w = 0;
            d3_vals[ID_DENS] = 0;
        }
        const float rw = __fmul_rn(r, w);
        float flux[kMwVars];
        flux[ID_DENS] = __fsub_rn(rw, d3_vals[ID_DENS]);  // from the rounded product, as along x
        flux[ID_UMOM] = __fmaf_rn(rw, u, -d3_vals[ID_UMOM]);
        flux[ID_WMOM] = __fsub_rn(__fmaf_rn(rw, w, pr), d3_vals[ID_WMOM]);
        flux[ID_RHOT] = __fmaf_rn(rw, t, -d3_vals[ID_RHOT]);
        if (j > 0) {
            // Cell row k-1, whose forcing values are win[.][1] (array row k+1).  When the reference
            // runs this stage with forcing and out in one array (the second Runge-Kutta stage) its
            // gravity term reads the density the same launch has already updated: its threads are
            // numbered variable-major (:322-324) and the density blocks run far ahead of the
            // momentum blocks.  `gravity_from_out` selects that value here, where out is a
            // separate array.
            float dens_new = 0.f;
#pragma unroll
            for (int ll = 0; ll < kMwVars; ++ll) {
                float tend = __fdiv_rn(-__fsub_rn(flux[ll], below[ll]), p.dz);
                if (ll == ID_WMOM) tend = __fmaf_rn(-(p.gravity_from_out ? dens_new : win[ID_DENS][1]), kGrav, tend);
                const float v = advance(init_v[ll], p.dt, tend);
                if (ll == ID_DENS) dens_new = v;
                p.out[ll * g.plane + cell] = v;
            }
        }
#pragma unroll
        for (int ll = 0; ll < kMwVars; ++ll) below[ll] = flux[ll];
    }
}

constexpr int kStageFloats = kMwVars * (kMwTileXMax + 2 * kMwHalo) + kMwVars * (kMwTileXMax + 1);

}  // namespace

// One kernel per direction, so each gets its own register budget (the x direction holds doubles
// and a staged row, the z direction a 4 x 4 stencil window and two prefetched rows).
template <int DIR>
__global__ void __launch_bounds__(kMwThreads, 4)
miniweather_step_kernel(const __grid_constant__ StencilParams p, BlpArgs blp) {
    pdl_enter();
    __shared__ float smem[DIR == 1 ? kStageFloats : 1];
    __shared__ int s_tile;
    const bool dynamic = blp.preempted != nullptr;
    if (threadIdx.x == 0) trace_begin(blp);
    const Grid g = grid_of(p);
    int iter = 0;
    for (;;) {
        int tile;
        if (dynamic) {
            __syncthreads();  // every thread has read the previous s_tile
            if (threadIdx.x == 0) s_tile = blp_claim(blp, iter);
            __syncthreads();
            tile = s_tile;
        } else {
            tile = blp_claim(blp, iter);
        }
        if (tile < 0) break;
        if (DIR == 1) {
            tile_x(p, g, tile, smem);
            __syncthreads();  // the staging area is reused by the next tile
        } else {
            tile_z(p, g, tile);
        }
        ++iter;
    }
    if (threadIdx.x == 0) trace_end(blp, iter);
}

namespace {

// ---- initial state (sci_init, miniweather.cu:376-507) --------------------------------------

// hydro_const_theta (:580-590): hydrostatic balance at constant potential temperature.
void hydro_const_theta(float z, float &r, float &t) {
    const float theta0 = 300.;
    const float exner0 = 1.;
    float p, exner, rt;
    t = theta0;
    exner = exner0 - kGrav * z / (kCp * theta0);
    p = kP0 * std::pow(exner, (kCp / kRd));
    rt = std::pow((p / kC0), (1. / kGamm));
    r = rt / t;
}

// sample_ellipse_cosine (:612-622).
float sample_ellipse_cosine(float x, float z, float amp, float x0, float z0, float xrad, float zrad) {
    float dist = std::sqrt(((x - x0) / xrad) * ((x - x0) / xrad) + ((z - z0) / zrad) * ((z - z0) / zrad)) * kPi / 2.;
    if (dist <= kPi / 2.) return amp * std::pow(std::cos(dist), 2.);
    return 0.;
}

// collision (:566-575): two thermals of opposite sign on one vertical line.
void collision(float x, float z, float &r, float &u, float &w, float &t, float &hr, float &ht) {
    hydro_const_theta(z, hr, ht);
    r = 0.;
    t = 0.;
    u = 0.;
    w = 0.;
    t = t + sample_ellipse_cosine(x, z, 20., kXlen / 2, 2000., 2000., 2000.);
    t = t + sample_ellipse_cosine(x, z, -20., kXlen / 2, 8000., 2000., 2000.);
}

constexpr int kQ = 3;
constexpr float kQPoints[kQ] = {0.112701665379258311482073460022E0, 0.500000000000000000000000000000E0,
                                0.887298334620741688517926539980E0};
constexpr float kQWeights[kQ] = {0.277777777777777777777777777779E0, 0.444444444444444444444444444444E0,
                                 0.277777777777777777777777777779E0};

struct HostFields {
    std::vector<float> state, hy_dens_cell, hy_dens_theta_cell, hy_dens_int, hy_dens_theta_int, hy_pressure_int;
};

void init_rows(HostFields &h, int nx, int nz, float dx, float dz, int k_from, int k_to) {
    const int W = nx + 2 * kMwHalo;
    const size_t plane = (size_t)(nz + 2 * kMwHalo) * W;
    for (int k = k_from; k < k_to; ++k)
        for (int i = 0; i < W; ++i) {
            float acc[kMwVars] = {0.f, 0.f, 0.f, 0.f};
            for (int kk = 0; kk < kQ; ++kk)
                for (int ii = 0; ii < kQ; ++ii) {
                    float x = (0 + i - kMwHalo + 0.5) * dx + (kQPoints[ii] - 0.5) * dx;
                    float z = (0 + k - kMwHalo + 0.5) * dz + (kQPoints[kk] - 0.5) * dz;
                    float r, u, w, t, hr, ht;
                    collision(x, z, r, u, w, t, hr, ht);
                    acc[ID_DENS] = acc[ID_DENS] + r * kQWeights[ii] * kQWeights[kk];
                    acc[ID_UMOM] = acc[ID_UMOM] + (r + hr) * u * kQWeights[ii] * kQWeights[kk];
                    acc[ID_WMOM] = acc[ID_WMOM] + (r + hr) * w * kQWeights[ii] * kQWeights[kk];
                    acc[ID_RHOT] = acc[ID_RHOT] + ((r + hr) * (t + ht) - hr * ht) * kQWeights[ii] * kQWeights[kk];
                }
            for (int ll = 0; ll < kMwVars; ++ll) h.state[ll * plane + (size_t)k * W + i] = acc[ll];
        }
}

void init_fields(HostFields &h, int nx, int nz, float dx, float dz) {
    const int W = nx + 2 * kMwHalo, R = nz + 2 * kMwHalo;
    h.state.assign((size_t)kMwVars * R * W, 0.f);
    unsigned nt = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < nt; ++t) {
        int a = (int)((long long)R * t / nt), b = (int)((long long)R * (t + 1) / nt);
        pool.emplace_back([&h, nx, nz, dx, dz, a, b] { init_rows(h, nx, nz, dx, dz, a, b); });
    }
    for (auto &t : pool) t.join();
    // Hydrostatic background over cells: every quadrature point samples the cell centre
    // (miniweather.cu:461-475 omits the quadrature offset of z).
    h.hy_dens_cell.assign(R, 0.f);
    h.hy_dens_theta_cell.assign(R, 0.f);
    for (int k = 0; k < R; ++k)
        for (int kk = 0; kk < kQ; ++kk) {
            float z = (0 + k - kMwHalo + 0.5) * dz;
            float r, u, w, t, hr, ht;
            collision(0., z, r, u, w, t, hr, ht);
            h.hy_dens_cell[k] = h.hy_dens_cell[k] + hr * kQWeights[kk];
            h.hy_dens_theta_cell[k] = h.hy_dens_theta_cell[k] + hr * ht * kQWeights[kk];
        }
    // ... and at the interfaces (:477-488).
    h.hy_dens_int.assign(nz + 1, 0.f);
    h.hy_dens_theta_int.assign(nz + 1, 0.f);
    h.hy_pressure_int.assign(nz + 1, 0.f);
    for (int k = 0; k < nz + 1; ++k) {
        float z = (0 + k) * dz;
        float r, u, w, t, hr, ht;
        collision(0., z, r, u, w, t, hr, ht);
        h.hy_dens_int[k] = hr;
        h.hy_dens_theta_int[k] = hr * ht;
        h.hy_pressure_int[k] = kC0 * std::pow((hr * ht), kGamm);
    }
}

int add_field(gpx_model &m, const char *name, Storage::Kind kind, int rank, int64_t d0, int64_t d1, int64_t d2,
              const float *host, bool hidden) {
    Storage s;
    s.name = name;
    s.kind = kind;
    s.rank = rank;
    s.dims[0] = d0;
    s.dims[1] = d1;
    s.dims[2] = d2;
    s.dims[3] = 1;
    size_t n = (size_t)d0 * (rank > 1 ? d1 : 1) * (rank > 2 ? d2 : 1);
    s.bytes = n * sizeof(float);
    s.hidden = hidden;
    GPX_CUDA(cudaMalloc((void **)&s.dptr, s.bytes));
    GPX_CUDA(cudaMemcpy(s.dptr, host, s.bytes, cudaMemcpyHostToDevice));
    m.add_storage(s);
    return GPX_SUCC;
}

}  // namespace

int stencil_grid(int dir, int total_tiles, int sm_count) {
    int blocks = 0;
    if (dir == 1)
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, miniweather_step_kernel<1>, kMwThreads, 0);
    else
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, miniweather_step_kernel<2>, kMwThreads, 0);
    if (blocks < 1) blocks = 1;
    long long grid = (long long)blocks * sm_count;
    if (grid > total_tiles) grid = total_tiles;
    return grid < 1 ? 1 : (int)grid;
}

cudaError_t stencil_launch(const StencilParams &p, int grid, const BlpArgs &blp, cudaStream_t s) {
    if (p.dir == 1)
        launch_layer(miniweather_step_kernel<1>, grid, kMwThreads, 0, s, p, blp);
    else
        launch_layer(miniweather_step_kernel<2>, grid, kMwThreads, 0, s, p, blp);
    return cudaGetLastError();
}

// "miniweather" is the reference's grid (3200 x 1600, miniweather.cu:21-22); "miniweather_tiny"
// (320 x 160) and "miniweather_<nx>x<nz>" exist for tests.
static bool parse_grid(const std::string &name, int &nx, int &nz) {
    if (name == "miniweather") {
        nx = 3200;
        nz = 1600;
        return true;
    }
    if (name == "miniweather_tiny") {
        nx = 320;
        nz = 160;
        return true;
    }
    int a = 0, b = 0;
    char tail = 0;
    if (sscanf(name.c_str(), "miniweather_%dx%d%c", &a, &b, &tail) == 2) {
        nx = a;
        nz = b;
        return true;
    }
    return false;
}

bool is_miniweather(const std::string &name) {
    int nx, nz;
    return parse_grid(name, nx, nz);
}

int build_miniweather(gpx_model &m, const std::string &name, const gpx_model_opts &) {
    int nx = 0, nz = 0;
    GPX_REQUIRE(parse_grid(name, nx, nz), GPX_NOT_FOUND, "unknown model '%s'", name.c_str());
    GPX_REQUIRE(nx >= 8 && nz >= 8 && nx <= 32768 && nz <= 32768 && (long long)nx * nz <= (1ll << 27), GPX_OUT_OF_RANGE,
                "%s: grid %d x %d is outside 8..32768 per side and 2^27 cells", name.c_str(), nx, nz);
    const DeviceInfo &d = device_info();
    GPX_REQUIRE(d.device >= 0, GPX_FAIL, "gpx_init was not called");
    m.device = d.device;
    m.sm_count = d.sm_count;
    m.sci = true;
    m.sci_nx = nx;
    m.sci_nz = nz;
    const float dx = kXlen / nx, dz = kZlen / nz;
    const float dt = std::min(dx, dz) / kMaxSpeed * kCfl;
    m.sci_dt = dt;
    m.sci_dx = dx;
    m.sci_dz = dz;

    HostFields h;
    init_fields(h, nx, nz, dx, dz);
    const int W = nx + 2 * kMwHalo, R = nz + 2 * kMwHalo;
    // state, state_tmp as the reference names them (:142-143); state_tmp2 receives the second
    // Runge-Kutta stage.  All three start from the initial state, halo cells included.
    GPX_TRY(add_field(m, "state", Storage::Table, 3, kMwVars, R, W, h.state.data(), false));
    GPX_TRY(add_field(m, "state_tmp", Storage::Table, 3, kMwVars, R, W, h.state.data(), false));
    GPX_TRY(add_field(m, "state_tmp2", Storage::Table, 3, kMwVars, R, W, h.state.data(), true));
    GPX_TRY(add_field(m, "hy_dens_cell", Storage::Vec, 1, R, 1, 1, h.hy_dens_cell.data(), false));
    GPX_TRY(add_field(m, "hy_dens_theta_cell", Storage::Vec, 1, R, 1, 1, h.hy_dens_theta_cell.data(), false));
    GPX_TRY(add_field(m, "hy_dens_int", Storage::Vec, 1, nz + 1, 1, 1, h.hy_dens_int.data(), false));
    GPX_TRY(add_field(m, "hy_dens_theta_int", Storage::Vec, 1, nz + 1, 1, 1, h.hy_dens_theta_int.data(), false));
    GPX_TRY(add_field(m, "hy_pressure_int", Storage::Vec, 1, nz + 1, 1, 1, h.hy_pressure_int.data(), false));
    m.sci_hy_dens_cell = h.hy_dens_cell;
    m.sci_hy_dens_theta_cell = h.hy_dens_theta_cell;
    m.sci_initial = std::move(h.state);

    StencilParams base{};
    base.hy_dens_cell = m.storages[m.find("hy_dens_cell")].dptr;
    base.hy_dens_theta_cell = m.storages[m.find("hy_dens_theta_cell")].dptr;
    base.hy_dens_int = m.storages[m.find("hy_dens_int")].dptr;
    base.hy_dens_theta_int = m.storages[m.find("hy_dens_theta_int")].dptr;
    base.hy_pressure_int = m.storages[m.find("hy_pressure_int")].dptr;
    // hy_dens_cell_const (:501-506)
    base.halo_ratio[0] = h.hy_dens_cell[0] / h.hy_dens_cell[kMwHalo];
    base.halo_ratio[1] = h.hy_dens_cell[1] / h.hy_dens_cell[kMwHalo];
    base.halo_ratio[2] = h.hy_dens_cell[nz + kMwHalo] / h.hy_dens_cell[nz + kMwHalo - 1];
    base.halo_ratio[3] = h.hy_dens_cell[nz + kMwHalo + 1] / h.hy_dens_cell[nz + kMwHalo - 1];
    base.dx = dx;
    base.dz = dz;
    base.nx = nx;
    base.nz = nz;
    const int row_tiles = (nx + kMwTileXMax - 1) / kMwTileXMax;
    base.tile_x = ((nx + row_tiles - 1) / row_tiles + 31) / 32 * 32;
    base.tiles_per_row = (nx + base.tile_x - 1) / base.tile_x;
    base.tiles_cols = (nx + kMwThreads - 1) / kMwThreads;
    // Rows per vertical tile: every tile recomputes one flux row and re-reads three stencil rows,
    // so taller is cheaper, but the static schedule of a non-preemptible executor gives each CTA
    // ceil(tiles / grid) tiles; pick the height that wastes least of both.
    {
        const int grid_full = stencil_grid(2, 1 << 30, m.sm_count);
        double best = -1.0;
        for (int rows = 8; rows <= kMwTileZRowsMax; ++rows) {
            const long long tiles = (long long)base.tiles_cols * ((nz + rows - 1) / rows);
            const long long waves = (tiles + grid_full - 1) / grid_full;
            const double eff = (double)tiles / (double)(waves * std::min<long long>(grid_full, tiles)) * rows / (rows + 1.5);
            if (eff > best) {
                best = eff;
                base.tile_rows = rows;
            }
        }
    }
    const char *cover = getenv("GPX_MINIWEATHER_FULL_HALO");
    base.halo_z_ids = (cover && cover[0] == '1') ? W * kMwVars
                                                 : (nx + 2 * kMwHalo * kMwVars + 255) / 256 * 256;

    float *state = m.storages[m.find("state")].dptr;
    float *tmp = m.storages[m.find("state_tmp")].dptr;
    float *tmp2 = m.storages[m.find("state_tmp2")].dptr;
    // perform_timestep (:182-200): x, z, z, x, each a three-stage Runge-Kutta sweep.
    const int dirs[4] = {1, 2, 2, 1};
    for (int sweep = 0; sweep < 4; ++sweep)
        for (int stage = 0; stage < 3; ++stage) {
            Kernel k;
            k.type = KernelType::Stencil;
            k.name = std::string("miniweather_step_kernel.") + (dirs[sweep] == 1 ? "x" : "z") + std::to_string(sweep) +
                     ".rk" + std::to_string(stage + 1);
            StencilParams p = base;
            p.dir = dirs[sweep];
            p.init = state;
            p.forcing = stage == 0 ? state : (stage == 1 ? tmp : tmp2);
            p.out = stage == 0 ? tmp : (stage == 1 ? tmp2 : state);
            p.dt = stage == 0 ? dt / 3 : (stage == 1 ? dt / 2 : dt / 1);
            p.gravity_from_out = stage == 1 ? 1 : 0;
            k.stencil = p;
            k.threads = kMwThreads;
            k.total_tiles = p.dir == 1 ? nz * p.tiles_per_row
                                       : p.tiles_cols * ((nz + p.tile_rows - 1) / p.tile_rows);
            k.grid = stencil_grid(p.dir, k.total_tiles, m.sm_count);
            const double cells = (double)nx * nz;
            k.bytes = cells * kMwVars * 4.0 * 3.0;  // forcing and init read, out written
            k.flops = cells * (p.dir == 1 ? 120.0 : 100.0);
            m.kernels.push_back(k);
        }
    return GPX_SUCC;
}

}  // namespace gpx

extern "C" {

// reductions (miniweather.cu:650-677): domain mass and total energy in double from the float state.
int gpx_model_reductions(gpx_model *m, double *mass, double *te) {
    using namespace gpx;
    GPX_REQUIRE(m && mass && te, GPX_FAIL, "NULL argument");
    GPX_REQUIRE(m->sci && m->graph_algo < 0, GPX_NOT_FOUND, "model '%s' has no reductions (miniweather only)", m->name.c_str());
    const int nx = m->sci_nx, nz = m->sci_nz, W = nx + 2 * kMwHalo;
    const size_t plane = (size_t)(nz + 2 * kMwHalo) * W;
    std::vector<float> st(plane * kMwVars);
    GPX_CUDA(cudaMemcpy(st.data(), m->storages[m->find("state")].dptr, st.size() * sizeof(float),
                        cudaMemcpyDeviceToHost));
    double ms = 0, en = 0;
    const float dx = m->sci_dx, dz = m->sci_dz;
    for (int k = 0; k < nz; ++k)
        for (int i = 0; i < nx; ++i) {
            size_t at = (size_t)(k + kMwHalo) * W + i + kMwHalo;
            double r = st[ID_DENS * plane + at] + m->sci_hy_dens_cell[kMwHalo + k];
            double u = st[ID_UMOM * plane + at] / r;
            double w = st[ID_WMOM * plane + at] / r;
            double th = (st[ID_RHOT * plane + at] + m->sci_hy_dens_theta_cell[kMwHalo + k]) / r;
            double p = kC0 * pow(r * th, kGamm);
            double t = th / pow(kP0 / p, kRd / kCp);
            double ke = r * (u * u + w * w);
            double ie = r * kCv * t;
            ms += r * dx * dz;
            en += (ke + ie) * dx * dz;
        }
    *mass = ms;
    *te = en;
    return GPX_SUCC;
}

}  // extern "C"
