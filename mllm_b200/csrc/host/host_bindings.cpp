// Python binding of the host-side native components: KV slot allocator, radix prefix tree and the
// `.mllm` parameter-file reader / writer.  Arrays cross the boundary as numpy arrays; tensors of a
// mapped file are exposed without a copy (the array keeps the file object alive).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <memory>

#include "host/cpu_oracle.h"
#include "host/mllm_file.h"
#include "host/page_allocator.h"
#include "host/radix_tree.h"
#include "host/symm_heap.h"

namespace py = pybind11;
using namespace mb200host;

using I64Array = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;

static py::array_t<int64_t> to_array(const std::vector<int64_t>& v) {
  py::array_t<int64_t> a(static_cast<py::ssize_t>(v.size()));
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(int64_t));
  return a;
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<SymmHeapAllocator>(m, "SymmHeapAllocator")
      .def(py::init<int64_t, int64_t>(), py::arg("capacity"), py::arg("min_align") = 256)
      .def("alloc", &SymmHeapAllocator::alloc, py::arg("bytes"), py::arg("align") = 0)
      .def("free", &SymmHeapAllocator::free_block)
      .def("reset", &SymmHeapAllocator::reset)
      .def("block_size", &SymmHeapAllocator::block_size)
      .def_property_readonly("capacity", &SymmHeapAllocator::capacity)
      .def_property_readonly("used", &SymmHeapAllocator::used)
      .def_property_readonly("largest_free", &SymmHeapAllocator::largest_free)
      .def_property_readonly("num_blocks", &SymmHeapAllocator::num_blocks);

  py::class_<PageAllocator>(m, "PageAllocator")
      .def(py::init<int64_t, int>(), py::arg("num_slots"), py::arg("page_size") = 1)
      .def("clear", &PageAllocator::clear)
      .def("available", &PageAllocator::available)
      .def("alloc",
           [](PageAllocator& self, int64_t n) -> py::object {
             std::vector<int64_t> out;
             if (!self.alloc(n, &out)) return py::none();
             return to_array(out);
           })
      .def("free", [](PageAllocator& self, I64Array slots) { self.free_slots(slots.data(), slots.size()); })
      .def("group_begin", &PageAllocator::group_begin)
      .def("group_end", &PageAllocator::group_end)
      .def_property_readonly("page_size", &PageAllocator::page_size)
      .def_property_readonly("num_slots", &PageAllocator::num_slots);

  py::class_<RadixTree>(m, "RadixTree")
      .def(py::init<int>(), py::arg("page_size") = 1)
      .def("reset", &RadixTree::reset)
      .def("match_prefix",
           [](RadixTree& self, I64Array tokens, int64_t extra_key) {
             RadixMatch r = self.match_prefix(tokens.data(), tokens.size(), extra_key);
             return py::make_tuple(to_array(r.slots), r.node);
           },
           py::arg("tokens"), py::arg("extra_key") = 0)
      .def("insert",
           [](RadixTree& self, I64Array tokens, I64Array slots, int64_t extra_key) {
             if (slots.size() < tokens.size()) throw std::invalid_argument("insert: fewer slots than tokens");
             int64_t last = 0;
             const int64_t matched = self.insert(tokens.data(), slots.data(), tokens.size(), extra_key, &last);
             return py::make_tuple(matched, last);
           },
           py::arg("tokens"), py::arg("slots"), py::arg("extra_key") = 0)
      .def("inc_lock_ref", &RadixTree::inc_lock)
      .def("dec_lock_ref", &RadixTree::dec_lock)
      .def("evict", [](RadixTree& self, int64_t n) { return to_array(self.evict(n)); })
      .def("evictable_size", &RadixTree::evictable_size)
      .def("protected_size", &RadixTree::protected_size)
      .def("total_size", &RadixTree::total_size)
      .def("num_nodes", &RadixTree::num_nodes)
      .def("dump", [](const RadixTree& self) {
        py::list out;
        for (const auto& n : self.dump()) out.append(py::make_tuple(n.id, n.parent, n.lock_ref, n.last_access, n.key));
        return out;
      });

  py::class_<MllmFile, std::shared_ptr<MllmFile>>(m, "MllmFile")
      .def(py::init<const std::string&>())
      .def_property_readonly("version", &MllmFile::version)
      .def_property_readonly("model_name", &MllmFile::model_name)
      .def("names",
           [](const MllmFile& f) {
             std::vector<std::string> out;
             for (const auto& p : f.params()) out.push_back(p.name);
             return out;
           })
      .def("info",
           [](const MllmFile& f, const std::string& name) {
             const MllmParam* p = f.find(name);
             if (p == nullptr) throw py::key_error(name);
             return py::make_tuple(p->dtype, p->shape, p->size, p->offset);
           })
      // raw bytes of a tensor as a read-only uint8 view of the mapping
      .def("raw",
           [](std::shared_ptr<MllmFile> f, const std::string& name) {
             const MllmParam* p = f->find(name);
             if (p == nullptr) throw py::key_error(name);
             py::object owner = py::cast(f);
             py::array_t<uint8_t> a({static_cast<py::ssize_t>(p->size)}, {1}, f->data(*p), owner);
             py::detail::array_proxy(a.ptr())->flags &= ~py::detail::npy_api::NPY_ARRAY_WRITEABLE_;
             return a;
           })
      // fp32 expansion of a GGUF block-quantised tensor
      .def("dequantize",
           [](const MllmFile& f, const std::string& name, int threads) {
             const MllmParam* p = f.find(name);
             if (p == nullptr) throw py::key_error(name);
             const int64_t n = gguf_num_elements(p->dtype, p->size);
             if (n <= 0) throw std::invalid_argument("dequantize: " + name + " is not a supported GGUF block format");
             py::array_t<float> out(n);
             float* dst = out.mutable_data();
             const uint8_t* src = f.data(*p);
             {
               py::gil_scoped_release rel;
               gguf_dequantize(p->dtype, src, p->size, dst, threads);
             }
             return out;
           },
           py::arg("name"), py::arg("threads") = 0);

  m.def("gguf_dequantize",
        [](int dtype, py::array_t<uint8_t, py::array::c_style | py::array::forcecast> raw, int threads) {
          const int64_t n = gguf_num_elements(dtype, raw.size());
          if (n <= 0) throw std::invalid_argument("gguf_dequantize: unsupported dtype or size");
          py::array_t<float> out(n);
          gguf_dequantize(dtype, raw.data(), raw.size(), out.mutable_data(), threads);
          return out;
        },
        py::arg("dtype"), py::arg("raw"), py::arg("threads") = 0);

  m.def("qwen3_cpu_generate",
        [](const std::string& path, py::dict cfg, std::vector<int64_t> prompt, int new_tokens, int threads) {
          OracleConfig c;
          c.vocab = cfg["vocab_size"].cast<int>();
          c.hidden = cfg["hidden_size"].cast<int>();
          c.inter = cfg["intermediate_size"].cast<int>();
          c.layers = cfg["num_hidden_layers"].cast<int>();
          c.heads = cfg["num_attention_heads"].cast<int>();
          c.kv_heads = cfg["num_key_value_heads"].cast<int>();
          c.head_dim = cfg["head_dim"].cast<int>();
          c.eps = cfg["rms_norm_eps"].cast<float>();
          c.theta = cfg["rope_theta"].cast<float>();
          c.tie = cfg["tie_word_embeddings"].cast<bool>();
          OracleResult r;
          {
            py::gil_scoped_release rel;
            r = qwen3_cpu_generate(path, c, prompt, new_tokens, threads);
          }
          py::dict out;
          out["tokens"] = r.tokens;
          out["prefill_logits"] = py::array_t<float>(r.prefill_logits.size(), r.prefill_logits.data());
          out["last_logits"] = py::array_t<float>(r.last_logits.size(), r.last_logits.data());
          out["prefill_seconds"] = r.prefill_seconds;
          out["decode_seconds"] = r.decode_seconds;
          return out;
        },
        py::arg("mllm_path"), py::arg("config"), py::arg("prompt"), py::arg("new_tokens"), py::arg("threads") = 0);

  m.def("write_mllm_v2",
        [](const std::string& path, const std::string& model_name, py::list entries) {
          std::vector<MllmWriteEntry> es;
          std::vector<py::array> keep;
          for (auto item : entries) {
            auto t = item.cast<py::tuple>();  // (name, dtype id, shape, uint8 array)
            auto arr = py::array_t<uint8_t, py::array::c_style | py::array::forcecast>::ensure(t[3]);
            if (!arr) throw std::invalid_argument("write_mllm_v2: data must be a uint8 array");
            keep.push_back(arr);
            MllmWriteEntry e;
            e.name = t[0].cast<std::string>();
            e.dtype = t[1].cast<int32_t>();
            e.shape = t[2].cast<std::vector<int32_t>>();
            e.data = static_cast<const uint8_t*>(arr.data());
            e.size = static_cast<uint64_t>(arr.size());
            es.push_back(std::move(e));
          }
          write_mllm_v2(path, model_name, es);
        });
}
