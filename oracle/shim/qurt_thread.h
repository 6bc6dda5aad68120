/* Host stand-in for the QuRT header of the same name (types only). */
#ifndef ORACLE_SHIM_QURT_THREAD_H
#define ORACLE_SHIM_QURT_THREAD_H
typedef int qurt_thread_t;
#endif
