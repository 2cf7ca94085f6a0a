/* CPU restatement of the reference's miniWeather workload - TEST INFRASTRUCTURE ONLY.
 *
 * Only tests/, the smoke check and bench.py's CPU baseline may load this library; the product
 * never does.  Pinned: tests/test_gpu_miniweather.py compares it with the reference's own
 * kernels (src/workloads/miniweather.cu compiled unmodified into oracle/_ref by the Makefile's
 * `ref` target) after time steps on the reference's 3200 x 1600 grid, and
 * tests/golden/miniweather_*.json holds figures produced by that code.
 *
 * Structure follows the reference, not the product: two state arrays, a flux array in memory and
 * three passes per semi-discrete step (halo, flux, update).  Arithmetic types follow the
 * reference's expressions: `real` is float, the horizontal flux works in double
 * (miniweather.cu:243-248), and mixed float/double sub-expressions are written out with the
 * conversions C++ would apply.  Compiled with -ffp-contract=off; the GPU code contracts
 * multiply-adds, so comparisons with it carry a tolerance.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#define HS 2
#define NUM_VARS 4
#define ID_DENS 0
#define ID_UMOM 1
#define ID_WMOM 2
#define ID_RHOT 3

/* miniweather.cu:35-47 */
static const float pi = 3.14159265358979323846264338327;
static const float grav = 9.8;
static const float cp = 1004.;
static const float cv = 717.;
static const float rd = 287.;
static const float p0 = 1.e5;
static const float C0 = 27.5629410929725921310572974482;
static const float gamm = 1.40027894002789400278940027894;
static const float xlen = 2.e4;
static const float zlen = 1.e4;
static const float hv_beta = 0.05;
static const float cfl = 1.50;
static const float max_speed = 450;

static const float qpoints[3] = {0.112701665379258311482073460022E0, 0.500000000000000000000000000000E0,
                                 0.887298334620741688517926539980E0};
static const float qweights[3] = {0.277777777777777777777777777779E0, 0.444444444444444444444444444444E0,
                                  0.277777777777777777777777777779E0};

typedef struct {
    int nx, nz;
    float dx, dz, dt;
    float *state, *state_tmp, *flux;
    float *hy_dens_cell, *hy_dens_theta_cell, *hy_dens_int, *hy_dens_theta_int, *hy_pressure_int;
    float hy_const[4];
    int halo_z_ids; /* threads of the reference's vertical halo launch (miniweather.cu:213) */
} mwo;

/* hydro_const_theta, miniweather.cu:580-590 */
static void hydro_const_theta(float z, float *r, float *t) {
    const float theta0 = 300.;
    const float exner0 = 1.;
    float p, exner, rt;
    *t = theta0;
    exner = exner0 - grav * z / (cp * theta0);
    p = p0 * powf(exner, (cp / rd));
    rt = (float)pow((double)(p / C0), (1. / (double)gamm));
    *r = rt / *t;
}

/* sample_ellipse_cosine, miniweather.cu:612-622 */
static float sample_ellipse_cosine(float x, float z, float amp, float x0, float z0, float xrad, float zrad) {
    float dist = (float)((double)(sqrtf(((x - x0) / xrad) * ((x - x0) / xrad) + ((z - z0) / zrad) * ((z - z0) / zrad)) * pi) / 2.);
    if ((double)dist <= (double)pi / 2.) return (float)((double)amp * pow((double)cosf(dist), 2.));
    return 0.f;
}

/* collision, miniweather.cu:566-575 */
static void collision(float x, float z, float *r, float *u, float *w, float *t, float *hr, float *ht) {
    hydro_const_theta(z, hr, ht);
    *r = 0.f;
    *t = 0.f;
    *u = 0.f;
    *w = 0.f;
    *t = *t + sample_ellipse_cosine(x, z, 20.f, xlen / 2, 2000.f, 2000.f, 2000.f);
    *t = *t + sample_ellipse_cosine(x, z, -20.f, xlen / 2, 8000.f, 2000.f, 2000.f);
}

void mwo_destroy(mwo *m) {
    if (!m) return;
    free(m->state);
    free(m->state_tmp);
    free(m->flux);
    free(m->hy_dens_cell);
    free(m->hy_dens_theta_cell);
    free(m->hy_dens_int);
    free(m->hy_dens_theta_int);
    free(m->hy_pressure_int);
    free(m);
}

/* sci_init, miniweather.cu:376-507.  full_halo != 0 lets the vertical halo pass cover every
 * variable instead of the reference's thread count. */
mwo *mwo_create(int nx, int nz, int full_halo) {
    mwo *m = (mwo *)calloc(1, sizeof(mwo));
    const int W = nx + 2 * HS, R = nz + 2 * HS;
    const size_t plane = (size_t)R * W;
    m->nx = nx;
    m->nz = nz;
    m->dx = xlen / nx;
    m->dz = zlen / nz;
    m->dt = (m->dx < m->dz ? m->dx : m->dz) / max_speed * cfl;
    m->halo_z_ids = full_halo ? W * NUM_VARS : (nx + 2 * HS * NUM_VARS + 255) / 256 * 256;
    m->state = (float *)calloc(plane * NUM_VARS, sizeof(float));
    m->state_tmp = (float *)calloc(plane * NUM_VARS, sizeof(float));
    m->flux = (float *)calloc((size_t)(nx + 1) * (nz + 1) * NUM_VARS, sizeof(float));
    m->hy_dens_cell = (float *)calloc(R, sizeof(float));
    m->hy_dens_theta_cell = (float *)calloc(R, sizeof(float));
    m->hy_dens_int = (float *)calloc(nz + 1, sizeof(float));
    m->hy_dens_theta_int = (float *)calloc(nz + 1, sizeof(float));
    m->hy_pressure_int = (float *)calloc(nz + 1, sizeof(float));
    const float dx = m->dx, dz = m->dz;
#pragma omp parallel for schedule(static)
    for (int k = 0; k < R; k++)
        for (int i = 0; i < W; i++) {
            float acc[NUM_VARS] = {0.f, 0.f, 0.f, 0.f};
            for (int kk = 0; kk < 3; kk++)
                for (int ii = 0; ii < 3; ii++) {
                    float x = (float)((0 + i - HS + 0.5) * (double)dx + ((double)qpoints[ii] - 0.5) * (double)dx);
                    float z = (float)((0 + k - HS + 0.5) * (double)dz + ((double)qpoints[kk] - 0.5) * (double)dz);
                    float r, u, w, t, hr, ht;
                    collision(x, z, &r, &u, &w, &t, &hr, &ht);
                    acc[ID_DENS] = acc[ID_DENS] + r * qweights[ii] * qweights[kk];
                    acc[ID_UMOM] = acc[ID_UMOM] + (r + hr) * u * qweights[ii] * qweights[kk];
                    acc[ID_WMOM] = acc[ID_WMOM] + (r + hr) * w * qweights[ii] * qweights[kk];
                    acc[ID_RHOT] = acc[ID_RHOT] + ((r + hr) * (t + ht) - hr * ht) * qweights[ii] * qweights[kk];
                }
            for (int ll = 0; ll < NUM_VARS; ll++) {
                m->state[ll * plane + (size_t)k * W + i] = acc[ll];
                m->state_tmp[ll * plane + (size_t)k * W + i] = acc[ll];
            }
        }
    for (int k = 0; k < R; k++)
        for (int kk = 0; kk < 3; kk++) {
            float z = (float)((0 + k - HS + 0.5) * (double)dz);
            float r, u, w, t, hr, ht;
            collision(0.f, z, &r, &u, &w, &t, &hr, &ht);
            m->hy_dens_cell[k] = m->hy_dens_cell[k] + hr * qweights[kk];
            m->hy_dens_theta_cell[k] = m->hy_dens_theta_cell[k] + hr * ht * qweights[kk];
        }
    for (int k = 0; k < nz + 1; k++) {
        float z = (0 + k) * dz;
        float r, u, w, t, hr, ht;
        collision(0.f, z, &r, &u, &w, &t, &hr, &ht);
        m->hy_dens_int[k] = hr;
        m->hy_dens_theta_int[k] = hr * ht;
        m->hy_pressure_int[k] = C0 * powf((hr * ht), gamm);
    }
    m->hy_const[0] = m->hy_dens_cell[0] / m->hy_dens_cell[HS];
    m->hy_const[1] = m->hy_dens_cell[1] / m->hy_dens_cell[HS];
    m->hy_const[2] = m->hy_dens_cell[nz + HS] / m->hy_dens_cell[nz + HS - 1];
    m->hy_const[3] = m->hy_dens_cell[nz + HS + 1] / m->hy_dens_cell[nz + HS - 1];
    return m;
}

/* set_halo_values_x, miniweather.cu:331-341 */
static void halo_x(const mwo *m, float *state) {
    const int nx = m->nx, nz = m->nz, W = nx + 2 * HS;
    const size_t plane = (size_t)(nz + 2 * HS) * W;
    for (int ll = 0; ll < NUM_VARS; ll++)
        for (int k = 0; k < nz; k++) {
            float *row = state + ll * plane + (size_t)(k + HS) * W;
            row[0] = row[nx + HS - 2];
            row[1] = row[nx + HS - 1];
            row[nx + HS] = row[HS];
            row[nx + HS + 1] = row[HS + 1];
        }
}

/* set_halo_values_z, miniweather.cu:346-372, for the thread ids the launch at :213 creates */
static void halo_z(const mwo *m, float *state) {
    const int nx = m->nx, nz = m->nz, W = nx + 2 * HS;
    const size_t plane = (size_t)(nz + 2 * HS) * W;
    for (int id = 0; id < m->halo_z_ids; id++) {
        int i = id % W, ll = id / W;
        if (ll >= NUM_VARS) continue;
        float *v = state + ll * plane;
        if (ll == ID_WMOM) {
            v[(size_t)0 * W + i] = 0.f;
            v[(size_t)1 * W + i] = 0.f;
            v[(size_t)(nz + HS) * W + i] = 0.f;
            v[(size_t)(nz + HS + 1) * W + i] = 0.f;
        } else if (ll == ID_UMOM) {
            v[(size_t)0 * W + i] = v[(size_t)HS * W + i] * m->hy_const[0];
            v[(size_t)1 * W + i] = v[(size_t)HS * W + i] * m->hy_const[1];
            v[(size_t)(nz + HS) * W + i] = v[(size_t)(nz + HS - 1) * W + i] * m->hy_const[2];
            v[(size_t)(nz + HS + 1) * W + i] = v[(size_t)(nz + HS - 1) * W + i] * m->hy_const[3];
        } else {
            v[(size_t)0 * W + i] = v[(size_t)HS * W + i];
            v[(size_t)1 * W + i] = v[(size_t)HS * W + i];
            v[(size_t)(nz + HS) * W + i] = v[(size_t)(nz + HS - 1) * W + i];
            v[(size_t)(nz + HS + 1) * W + i] = v[(size_t)(nz + HS - 1) * W + i];
        }
    }
}

/* compute_tendencies_x + compute_tendencies_x_r, miniweather.cu:222-272 */
static void step_x(const mwo *m, const float *init, const float *forcing, float *out, float dt) {
    const int nx = m->nx, nz = m->nz, W = nx + 2 * HS;
    const size_t plane = (size_t)(nz + 2 * HS) * W, fplane = (size_t)(nz + 1) * (nx + 1);
    float *flux = m->flux;
    const float dx = m->dx;
    const float hv_coef = -hv_beta * dx / (16 * dt);
#pragma omp parallel for schedule(static)
    for (int k = 0; k < nz; k++)
        for (int i = 0; i < nx + 1; i++) {
            float vals[NUM_VARS], d3_vals[NUM_VARS];
            for (int ll = 0; ll < NUM_VARS; ll++) {
                const float *s = forcing + ll * plane + (size_t)(k + HS) * W + i;
                vals[ll] = (-s[0] + 7 * (s[1] + s[2]) - s[3]) / 12;
                d3_vals[ll] = (-s[0] + 3 * (s[1] - s[2]) + s[3]) * hv_coef;
            }
            double r = (double)(vals[ID_DENS] + m->hy_dens_cell[k + HS]);
            double u = (double)vals[ID_UMOM] / r;
            double w = (double)vals[ID_WMOM] / r;
            double t = (double)(vals[ID_RHOT] + m->hy_dens_theta_cell[k + HS]) / r;
            double p = (double)C0 * pow((r * t), (double)gamm);
            flux[ID_DENS * fplane + (size_t)k * (nx + 1) + i] = (float)(r * u - (double)d3_vals[ID_DENS]);
            flux[ID_UMOM * fplane + (size_t)k * (nx + 1) + i] = (float)(r * u * u + p - (double)d3_vals[ID_UMOM]);
            flux[ID_WMOM * fplane + (size_t)k * (nx + 1) + i] = (float)(r * u * w - (double)d3_vals[ID_WMOM]);
            flux[ID_RHOT * fplane + (size_t)k * (nx + 1) + i] = (float)(r * u * t - (double)d3_vals[ID_RHOT]);
        }
#pragma omp parallel for schedule(static) collapse(2)
    for (int ll = 0; ll < NUM_VARS; ll++)
        for (int k = 0; k < nz; k++)
            for (int i = 0; i < nx; i++) {
                size_t f1 = ll * fplane + (size_t)k * (nx + 1) + i;
                float tend = -(flux[f1 + 1] - flux[f1]) / dx;
                size_t inds = ll * plane + (size_t)(k + HS) * W + i + HS;
                out[inds] = init[inds] + dt * tend;
            }
}

/* compute_tendencies_z + compute_tendencies_z_r, miniweather.cu:278-336 */
static void step_z(const mwo *m, const float *init, const float *forcing, float *out, float dt) {
    const int nx = m->nx, nz = m->nz, W = nx + 2 * HS;
    const size_t plane = (size_t)(nz + 2 * HS) * W, fplane = (size_t)(nz + 1) * (nx + 1);
    float *flux = m->flux;
    const float dz = m->dz;
    const float hv_coef = -hv_beta * dz / (16 * dt);
#pragma omp parallel for schedule(static)
    for (int k = 0; k < nz + 1; k++)
        for (int i = 0; i < nx; i++) {
            float vals[NUM_VARS], d3_vals[NUM_VARS];
            for (int ll = 0; ll < NUM_VARS; ll++) {
                const float *s = forcing + ll * plane + (size_t)k * W + i + HS;
                float s0 = s[0], s1 = s[W], s2 = s[2 * (size_t)W], s3 = s[3 * (size_t)W];
                vals[ll] = (-s0 + 7 * (s1 + s2) - s3) / 12;
                d3_vals[ll] = (-s0 + 3 * (s1 - s2) + s3) * hv_coef;
            }
            float r = vals[ID_DENS] + m->hy_dens_int[k];
            float u = vals[ID_UMOM] / r;
            float w = vals[ID_WMOM] / r;
            float t = (vals[ID_RHOT] + m->hy_dens_theta_int[k]) / r;
            float p = C0 * powf((r * t), gamm) - m->hy_pressure_int[k];
            if (k == 0 || k == nz) {
                w = 0;
                d3_vals[ID_DENS] = 0;
            }
            flux[ID_DENS * fplane + (size_t)k * (nx + 1) + i] = r * w - d3_vals[ID_DENS];
            flux[ID_UMOM * fplane + (size_t)k * (nx + 1) + i] = r * w * u - d3_vals[ID_UMOM];
            flux[ID_WMOM * fplane + (size_t)k * (nx + 1) + i] = r * w * w + p - d3_vals[ID_WMOM];
            flux[ID_RHOT * fplane + (size_t)k * (nx + 1) + i] = r * w * t - d3_vals[ID_RHOT];
        }
    /* In the second Runge-Kutta stage forcing and out are one array, and the reference's update
     * kernel reads the forcing density for the gravity term while other threads of the same launch
     * write the updated density.  Its threads are numbered variable-major (miniweather.cu:322-324),
     * so the density blocks run tens of thousands of blocks ahead of the vertical-momentum blocks:
     * the gravity term sees the updated density.  The variables are therefore updated one after
     * the other here, in that order. */
    for (int ll = 0; ll < NUM_VARS; ll++) {
#pragma omp parallel for schedule(static)
        for (int k = 0; k < nz; k++)
            for (int i = 0; i < nx; i++) {
                size_t f1 = ll * fplane + (size_t)k * (nx + 1) + i;
                float tend = -(flux[f1 + (nx + 1)] - flux[f1]) / dz;
                size_t at = (size_t)(k + HS) * W + i + HS;
                if (ll == ID_WMOM) tend = tend - forcing[ID_DENS * plane + at] * grav;
                size_t inds = ll * plane + at;
                out[inds] = init[inds] + dt * tend;
            }
    }
}

/* semi_discrete_step, miniweather.cu:204-216 */
static void semi_step(mwo *m, float *init, float *forcing, float *out, float dt, int dir) {
    if (dir == 1) {
        halo_x(m, forcing);
        step_x(m, init, forcing, out, dt);
    } else {
        halo_z(m, forcing);
        step_z(m, init, forcing, out, dt);
    }
}

/* perform_timestep, miniweather.cu:182-200.  `upto` (1..12) stops after that many semi-discrete
 * steps, for checks of the intermediate states. */
void mwo_timestep_upto(mwo *m, int upto) {
    static const int dirs[4] = {1, 2, 2, 1};
    float *state = m->state, *tmp = m->state_tmp;
    int n = 0;
    for (int sweep = 0; sweep < 4; sweep++) {
        if (n++ < upto) semi_step(m, state, state, tmp, m->dt / 3, dirs[sweep]);
        if (n++ < upto) semi_step(m, state, tmp, tmp, m->dt / 2, dirs[sweep]);
        if (n++ < upto) semi_step(m, state, tmp, state, m->dt / 1, dirs[sweep]);
    }
}

void mwo_timestep(mwo *m) { mwo_timestep_upto(m, 12); }

float *mwo_state(mwo *m) { return m->state; }
float *mwo_state_tmp(mwo *m) { return m->state_tmp; }
float *mwo_field(mwo *m, int which) {
    switch (which) {
        case 0: return m->hy_dens_cell;
        case 1: return m->hy_dens_theta_cell;
        case 2: return m->hy_dens_int;
        case 3: return m->hy_dens_theta_int;
        case 4: return m->hy_pressure_int;
        default: return m->hy_const;
    }
}
float mwo_dt(mwo *m) { return m->dt; }

/* reductions, miniweather.cu:650-677 */
void mwo_reductions(mwo *m, double *mass, double *te) {
    const int nx = m->nx, nz = m->nz, W = nx + 2 * HS;
    const size_t plane = (size_t)(nz + 2 * HS) * W;
    double ms = 0, en = 0;
    for (int k = 0; k < nz; k++)
        for (int i = 0; i < nx; i++) {
            size_t at = (size_t)(k + HS) * W + i + HS;
            double r = (double)(m->state[ID_DENS * plane + at] + m->hy_dens_cell[HS + k]);
            double u = (double)m->state[ID_UMOM * plane + at] / r;
            double w = (double)m->state[ID_WMOM * plane + at] / r;
            double th = (double)(m->state[ID_RHOT * plane + at] + m->hy_dens_theta_cell[HS + k]) / r;
            double p = (double)C0 * pow(r * th, (double)gamm);
            double t = th / pow((double)p0 / p, (double)(rd / cp));
            double ke = r * (u * u + w * w);
            double ie = r * (double)cv * t;
            ms += r * (double)m->dx * (double)m->dz;
            en += (ke + ie) * (double)m->dx * (double)m->dz;
        }
    *mass = ms;
    *te = en;
}
