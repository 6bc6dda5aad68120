/* Host stand-in for the QuRT header of the same name (types only). */
#ifndef ORACLE_SHIM_QURT_BARRIER_H
#define ORACLE_SHIM_QURT_BARRIER_H
typedef int qurt_barrier_t;
#endif
