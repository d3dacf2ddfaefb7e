// Minimal stand-in for ROOT's TBuffer.h, used ONLY to compile the reference generator sources
// (RModel.cxx, RModel_Base.cxx, SOFIE_common.cxx) into oracle/_ref without a ROOT installation.
// Test infrastructure: nothing in the product includes this file.
#ifndef ORACLE_ROOT_SHIM_TBUFFER
#define ORACLE_ROOT_SHIM_TBUFFER
typedef int Int_t;
class TBuffer {
public:
   bool IsReading() const { return false; }
};
struct OracleShimClass {
   template <class T> void ReadBuffer(TBuffer &, T *) {}
   template <class T> void WriteBuffer(TBuffer &, T *) {}
};
// The reference only needs Class()->ReadBuffer/WriteBuffer and a Streamer declaration.
#define ClassDefNV(name, ver)                                                       \
   static OracleShimClass *Class() { static OracleShimClass c; return &c; }         \
   void Streamer(TBuffer &);
#endif
