// SofieFunctor: wraps Session::infer of a generated model in a callable with one float argument per
// input feature and a slot number, the form a parallel event loop (RDataFrame) expects. Same interface
// as the reference's helper (src/SOFIE_core/inc/SOFIE/SOFIEHelpers.hxx:9-65):
//
//    auto f = SofieFunctor<7, SOFIE_mymodel::Session>(nslots, "mymodel.dat");
//    double y = f(slot, x0, x1, x2, x3, x4, x5, x6);      // first output of a batch-1 inference
//
// One Session per slot; a Session of the CUDA path owns a device context (stream, arena, uploaded
// weights, captured graph), so slots never share device state and calls on different slots may run
// on different threads. Calls on the same slot must not overlap (the reference has the same rule:
// a Session's intermediate tensors are shared between calls).
#ifndef SOFIE_SOFIE_HELPERS
#define SOFIE_SOFIE_HELPERS

#include <array>
#include <cstddef>
#include <memory>
#include <string>
#include <utility>
#include <vector>

template <typename I, typename F, typename T>
class SofieFunctorHelper;

template <std::size_t... N, typename Session_t, typename T>
class SofieFunctorHelper<std::index_sequence<N...>, Session_t, T> {
   template <std::size_t>
   using Arg = T; // expands to one T per index: operator() takes exactly sizeof...(N) features

   struct Slot {
      std::unique_ptr<Session_t> session;
      std::array<T, sizeof...(N)> input;
   };
   std::vector<Slot> fSlots;

public:
   SofieFunctorHelper(unsigned int nslots = 0, const std::string &filename = "")
   {
      // zero slots means a single Session (no parallel evaluation)
      fSlots.resize(nslots < 1 ? 1 : nslots);
      for (auto &s : fSlots) s.session = filename.empty() ? std::make_unique<Session_t>() : std::make_unique<Session_t>(filename);
   }

   double operator()(unsigned slot, Arg<N>... args)
   {
      Slot &s = fSlots.at(slot);
      s.input = {args...};
      return s.session->infer(s.input.data())[0];
   }

   std::size_t NSlots() const { return fSlots.size(); }
};

template <std::size_t N, typename Session_t>
auto SofieFunctor(unsigned int nslots = 0, const std::string &weightsFile = "")
   -> SofieFunctorHelper<std::make_index_sequence<N>, Session_t, float>
{
   return SofieFunctorHelper<std::make_index_sequence<N>, Session_t, float>(nslots, weightsFile);
}

#endif // SOFIE_SOFIE_HELPERS
