/* Host stand-in for the Hexagon SDK header of the same name: the reference
 * executor only needs a microsecond clock from it. Test infrastructure. */
#ifndef ORACLE_SHIM_HAP_PERF_H
#define ORACLE_SHIM_HAP_PERF_H
#include <stdint.h>
#include <time.h>
static inline int64_t HAP_perf_get_time_us(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (int64_t)ts.tv_sec * 1000000 + ts.tv_nsec / 1000;
}
#endif
