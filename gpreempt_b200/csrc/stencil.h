// miniWeather: the scientific best-effort workload of the reference (src/workloads/miniweather.cu,
// the block-level-preemptible variant src/workloads/miniweather.tr.cu; the task configs
// config/Y.json and config/R.json run it under a latency-critical DNN).  A dry, compressible,
// non-hydrostatic 2-D flow on an nx x nz grid with a 2-cell halo, four fluid variables, advanced
// by a dimensionally split three-stage Runge-Kutta step.  One `execute` is one time step.
#pragma once

#include <cuda_runtime.h>
#include <string>

#include "blp.cuh"

struct gpx_model;
struct gpx_model_opts;

namespace gpx {

constexpr int kMwHalo = 2;       // hs
constexpr int kMwVars = 4;       // rho', rho*u, rho*w, (rho*theta)'
constexpr int kMwThreads = 256;
constexpr int kMwTileXMax = 512; // cells of one row per x-direction tile (at most)
constexpr int kMwTileZRowsMax = 40;  // rows of a z-direction tile (chosen per grid); its columns are one per thread

// One semi-discrete step out = init + dt * rhs(forcing) in one direction (semi_discrete_step,
// src/workloads/miniweather.cu:204-216).  The reference runs it as three kernels (halo, flux,
// update) with the flux array in global memory; here one kernel computes the fluxes of a tile (in
// shared memory along x, in registers while walking down a column along z) and updates the tile,
// and the tiles on the domain edge produce (and store) the halo cells they read.  `out` never aliases `forcing`: the second Runge-Kutta stage writes a
// third state buffer instead of updating its forcing array in place.
struct StencilParams {
    const float *init;
    float *forcing;  // halo cells of this array are written by edge tiles
    float *out;
    const float *hy_dens_cell;        // [nz + 4]
    const float *hy_dens_theta_cell;  // [nz + 4]
    const float *hy_dens_int;         // [nz + 1]
    const float *hy_dens_theta_int;   // [nz + 1]
    const float *hy_pressure_int;     // [nz + 1]
    float halo_ratio[4];  // hy_dens_cell[{0, 1, nz+2, nz+3}] / hy_dens_cell[{2, 2, nz+1, nz+1}]
    float dt;             // stage step (dt/3, dt/2, dt)
    float dx, dz;
    int nx, nz;
    int dir;              // 1 = x, 2 = z
    int tile_x;           // x direction: cells per tile; tiles_per_row = ceil(nx / tile_x)
    int tiles_per_row;
    int tiles_cols;       // z direction: ceil(nx / kMwThreads)
    int tile_rows;        // z direction: rows per tile
    // The reference launches its vertical halo kernel with (nx + 2*hs*NUM_VARS + 255) / 256 blocks
    // (miniweather.cu:213), so only flat indices below that many threads get halo values: all of
    // the density and the first columns of the horizontal momentum.  The other vertical halo cells
    // keep the values the initial state gave them.  `halo_z_ids` is that thread count; a value of
    // (nx + 4) * 4 would cover every variable.
    int halo_z_ids;
    int gravity_from_out;  // vertical update: the gravity term reads the updated density (stage 2)
};

cudaError_t stencil_launch(const StencilParams &p, int grid, const BlpArgs &blp, cudaStream_t s);
int stencil_grid(int dir, int total_tiles, int sm_count);

bool is_miniweather(const std::string &name);
int build_miniweather(gpx_model &m, const std::string &name, const gpx_model_opts &opts);

}  // namespace gpx
