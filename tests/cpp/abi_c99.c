/* A C99 translation unit against the C ABI: the header must parse as plain C and every entry
 * point used here must link.  No device is needed: only calls that work without one are made. */
#include "gpx.h"

#include <stdio.h>
#include <string.h>

int main(void) {
    int tiles = 0;
    if (gpx_axpy_tiles(10000, 4096, &tiles) != GPX_SUCC || tiles != 3) return 1;
    if (strcmp(gpx_strerror(GPX_TIMEOUT), "Timeout") != 0) return 2;
    gpx_sched *s = NULL;
    if (gpx_sched_create(0, "blpclient", &s) != GPX_SUCC) return 3;
    int client = -1;
    if (gpx_sched_attach(s, NULL, 1, &client) != GPX_SUCC || client != 0) return 4;
    uint64_t ticket = 0;
    if (gpx_sched_enqueue(s, client, &ticket) != GPX_SUCC || ticket != 1) return 5;
    if (gpx_wait(s, client, ticket, 1000000) != GPX_TIMEOUT) return 6; /* nobody runs the dispatcher */
    if (gpx_sched_destroy(s) != GPX_SUCC) return 7;
    gpx_model_opts o;
    memset(&o, 0, sizeof(o));
    o.batch = 1;
    gpx_model *m = NULL;
    /* without a device this fails with a message instead of crashing */
    if (gpx_model_open("resnet_tiny", &o, &m) == GPX_SUCC) gpx_model_close(m);
    printf("PASS C99 client of gpx.h (%zu-byte gpx_blp)\n", sizeof(gpx_blp));
    return 0;
}
