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

#include <algorithm>
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

// SofieSharded: one batch across several GPUs of a box. The same idiom -- one Session per slot, nothing shared -- with a GPU
// per slot: the batch is cut into contiguous shards, one per device, every device runs its shard through its own Session
// (weights replicated when the Sessions are constructed), and the rows come back in batch order. The samples of a batch
// are independent on this path, so there is no exchange between devices and no collective.
//
//    SofieSharded<SOFIE_mymodel::Session> net("mymodel.dat", {0, 1, 2, 3}, /* largest batch */ 16384, /* floats per sample */ 4096);
//    std::vector<float> y = net.infer(batch, x);          // x: batch * 4096 floats on the host
//
// Session_t is a Session generated with a run-time batch parameter: Session(file, size_t) and infer(size_t, float*).
#include <exception>
#include <stdexcept>
#include <thread>

extern "C" int sofie_cuda_set_default_device(int device);

template <typename Session_t>
class SofieSharded {
   std::vector<std::unique_ptr<Session_t>> fSessions;
   std::vector<int> fDevices;
   std::size_t fShardMax = 0, fInPerSample = 0;

public:
   // devices: the CUDA device of every shard (a device may appear more than once); maxBatch: the largest batch infer()
   // will be given; inPerSample: floats of one sample of the model's input
   SofieSharded(const std::string &weightsFile, const std::vector<int> &devices, std::size_t maxBatch, std::size_t inPerSample)
      : fDevices(devices), fInPerSample(inPerSample)
   {
      if (devices.empty()) throw std::runtime_error("SofieSharded needs at least one device");
      fShardMax = (maxBatch + devices.size() - 1) / devices.size();
      if (fShardMax == 0) fShardMax = 1;
      for (int d : devices) {
         sofie_cuda_set_default_device(d); // the Session constructed next on this thread lives on device d
         try {
            fSessions.push_back(std::make_unique<Session_t>(weightsFile, fShardMax));
         } catch (...) {
            sofie_cuda_set_default_device(-1);
            throw;
         }
      }
      sofie_cuda_set_default_device(-1);
   }

   std::size_t NShards() const { return fSessions.size(); }
   // [begin, end) of shard g of a batch: ceil(batch / shards) samples each, the last ones may be short or empty
   std::pair<std::size_t, std::size_t> Bounds(std::size_t batch, std::size_t g) const
   {
      const std::size_t per = (batch + fSessions.size() - 1) / fSessions.size();
      const std::size_t b = std::min(batch, g * per);
      return {b, std::min(batch, b + per)};
   }

   std::vector<float> infer(std::size_t batch, float *x)
   {
      const std::size_t G = fSessions.size();
      if ((batch + G - 1) / G > fShardMax) throw std::runtime_error("SofieSharded: the batch is larger than the one the Sessions were constructed for");
      std::vector<std::vector<float>> parts(G);
      std::vector<std::exception_ptr> errors(G);
      std::vector<std::thread> workers;
      for (std::size_t g = 0; g < G; g++) {
         const auto range = Bounds(batch, g);
         if (range.first == range.second) continue;
         workers.emplace_back([&, g, range] {
            try {
               parts[g] = fSessions[g]->infer(range.second - range.first, x + range.first * fInPerSample);
            } catch (...) {
               errors[g] = std::current_exception();
            }
         });
      }
      for (auto &w : workers) w.join();
      for (auto &e : errors)
         if (e) std::rethrow_exception(e);
      std::size_t total = 0;
      for (auto &p : parts) total += p.size();
      std::vector<float> y;
      y.reserve(total);
      for (auto &p : parts) y.insert(y.end(), p.begin(), p.end());
      return y;
   }
};

#endif // SOFIE_SOFIE_HELPERS
