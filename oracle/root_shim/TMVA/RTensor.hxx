// Minimal row-major stand-in for TMVA::Experimental::RTensor, enough for the GNN helper
// declarations in the reference's SOFIE_common.hxx to compile. Test infrastructure only.
#ifndef ORACLE_ROOT_SHIM_RTENSOR
#define ORACLE_ROOT_SHIM_RTENSOR
#include <cstddef>
#include <memory>
#include <vector>
namespace TMVA { namespace Experimental {
enum class MemoryLayout { RowMajor = 1, ColumnMajor = 2 };
template <class T>
class RTensor {
   std::vector<std::size_t> fShape, fStrides;
   std::size_t fSize = 0;
   std::shared_ptr<std::vector<T>> fStore;
   MemoryLayout fLayout = MemoryLayout::RowMajor;
public:
   RTensor(std::vector<std::size_t> shape, MemoryLayout l = MemoryLayout::RowMajor) : fShape(shape), fLayout(l)
   {
      fSize = shape.empty() ? 0 : 1;
      for (auto s : shape) fSize *= s;
      fStrides.assign(shape.size(), 1);
      for (std::size_t i = shape.size(); i-- > 1;) fStrides[i - 1] = fStrides[i] * shape[i];
      fStore = std::make_shared<std::vector<T>>(fSize);
   }
   const std::vector<std::size_t> &GetShape() const { return fShape; }
   const std::vector<std::size_t> &GetStrides() const { return fStrides; }
   std::size_t GetSize() const { return fSize; }
   T *GetData() { return fStore->data(); }
   const T *GetData() const { return fStore->data(); }
   MemoryLayout GetMemoryLayout() const { return fLayout; }
   RTensor<T> Copy() const { RTensor<T> r(fShape, fLayout); *r.fStore = *fStore; return r; }
};
}}
#endif
