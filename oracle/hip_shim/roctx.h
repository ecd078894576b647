// ORACLE -- TEST INFRASTRUCTURE ONLY. Trace calls of the reference do nothing here.
#ifndef FTREF_ROCTX_H_
#define FTREF_ROCTX_H_
inline int roctxRangePushA(const char*) { return 0; }
inline int roctxRangePop() { return 0; }
inline void roctxMarkA(const char*) {}
#endif
