// Minimal stand-in for ROOT's TFile.h (ROOT-binary weight files are not usable through it).
// Test infrastructure: only used to compile the reference generator into oracle/_ref.
#ifndef ORACLE_ROOT_SHIM_TFILE
#define ORACLE_ROOT_SHIM_TFILE
#include <string>
struct OracleShimDir {
   int WriteObjectAny(const void *, const char *, const char *) { return 0; }
};
class TFile {
public:
   static TFile *Open(const char *, const char * = "") { return nullptr; }
   bool IsOpen() const { return false; }
   void *GetKey(const char *) { return nullptr; }
   void rmdir(const char *) {}
   OracleShimDir *mkdir(const char *) { static OracleShimDir d; return &d; }
   int Write(const char * = nullptr) { return 0; }
   void *Get(const char *) { return nullptr; }
};
#endif
