/* Host stand-in for the QuRT header of the same name (types only). */
#ifndef ORACLE_SHIM_QURT_MUTEX_H
#define ORACLE_SHIM_QURT_MUTEX_H
typedef int qurt_mutex_t;
#endif
