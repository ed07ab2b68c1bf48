// Minimal stand-in for the header of the reference's backend submodule that its
// Autotuner sources include but that is not part of the reference checkout. It declares
// only what Autotuner/src/Subkernel_distributions.cpp needs to compile: LOC_NUM,
// the message helpers and a LinkMap with reset_links(). Written from the call sites
// (Subkernel_distributions.cpp:15-19,318-320,354); contains no reference code.
// TEST INFRASTRUCTURE ONLY.
#ifndef ORACLE_REF_SHIM_LINKMAP_H
#define ORACLE_REF_SHIM_LINKMAP_H
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <list>
#include <string>

#ifndef LOC_NUM
#define LOC_NUM 9
#endif

inline void warning(const char* fmt, ...) { (void)fmt; }
inline void lprintf(short lvl, const char* fmt, ...) { (void)lvl; (void)fmt; }
inline void error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vfprintf(stderr, fmt, ap);
  va_end(ap);
  exit(42);
}
template <typename T>
inline const char* printlist(T*, int) { return ""; }
inline int idxize(int loc) { return loc == -1 ? LOC_NUM - 1 : loc; }
inline int deidxize(int idx) { return idx == LOC_NUM - 1 ? -1 : idx; }

typedef class LinkMap {
 public:
  void reset_links(int) {}
}* LinkMap_p;

#endif
