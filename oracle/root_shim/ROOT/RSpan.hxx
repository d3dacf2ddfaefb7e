// Stand-in for ROOT/RSpan.hxx: the reference only needs std::span.
#ifndef ORACLE_ROOT_SHIM_RSPAN
#define ORACLE_ROOT_SHIM_RSPAN
#include <span>
#endif
