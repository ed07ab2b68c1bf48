// Empty stand-in for a header of the reference's absent backend submodule; the
// distribution code needs nothing from it. TEST INFRASTRUCTURE ONLY.
#ifndef ORACLE_REF_SHIM_BACKEND_WRAPPERS_H
#define ORACLE_REF_SHIM_BACKEND_WRAPPERS_H
#endif
