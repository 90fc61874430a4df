// pybind11 surface of the checkpoint loaders: safetensors files exposed as zero-copy buffers.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/loaders.h"

namespace py = pybind11;
using namespace dgpp;
using namespace dgpp::loaders;

namespace {

py::dict info_dict(const TensorInfo& t) {
  py::dict d;
  d["name"] = t.name;
  d["dtype"] = t.dtype;
  d["shape"] = t.shape;
  d["nbytes"] = t.nbytes();
  return d;
}

// A read-only view of a tensor's bytes that keeps the mapping alive.
py::object tensor_view(const std::shared_ptr<SafetensorsFile>& f, const TensorInfo& t) {
  py::object owner = py::cast(f);
  return py::memoryview::from_memory(f->data(t), static_cast<py::ssize_t>(t.nbytes()));
}

}  // namespace

void bind_load(py::module_& m) {
  py::class_<SafetensorsFile, std::shared_ptr<SafetensorsFile>>(m, "SafetensorsFile")
      .def(py::init<const std::string&>())
      .def("path", &SafetensorsFile::path)
      .def("metadata", &SafetensorsFile::metadata)
      .def("names", [](const SafetensorsFile& f) {
        std::vector<std::string> n;
        for (const auto& t : f.tensors()) n.push_back(t.name);
        return n;
      })
      .def("info", [](const SafetensorsFile& f, const std::string& name) {
        const TensorInfo* t = f.find(name);
        if (!t) throw py::key_error(name);
        return info_dict(*t);
      })
      // bytes of a tensor as a read-only memoryview into the mapping (valid while the file object lives)
      .def("view", [](py::object self, const std::string& name) {
        auto f = self.cast<std::shared_ptr<SafetensorsFile>>();
        const TensorInfo* t = f->find(name);
        if (!t) throw py::key_error(name);
        py::object mv = tensor_view(f, *t);
        return py::make_tuple(mv, self);
      })
      .def("advise", [](const SafetensorsFile& f, const std::string& name, bool will_need) {
        const TensorInfo* t = f.find(name);
        if (!t) throw py::key_error(name);
        f.advise(*t, will_need);
      });

  m.def("write_safetensors", [](const std::string& path, const std::vector<std::tuple<std::string, std::string, std::vector<int64_t>, py::buffer>>& tensors,
                                const std::map<std::string, std::string>& metadata) {
    std::vector<TensorToWrite> tw;
    std::vector<py::buffer_info> keep;
    keep.reserve(tensors.size());
    for (const auto& t : tensors) {
      keep.push_back(std::get<3>(t).request());
      const auto& bi = keep.back();
      tw.push_back({std::get<0>(t), std::get<1>(t), std::get<2>(t), bi.ptr, static_cast<uint64_t>(bi.size * bi.itemsize)});
    }
    write_safetensors(path, tw, metadata);
  }, py::arg("path"), py::arg("tensors"), py::arg("metadata") = std::map<std::string, std::string>{});

  py::class_<Checkpoint>(m, "Checkpoint")
      .def(py::init<const std::string&>())
      .def("dir", &Checkpoint::dir)
      .def("names", &Checkpoint::names)
      .def("has", &Checkpoint::has)
      .def("info", [](Checkpoint& c, const std::string& name) { return info_dict(*c.get(name).second); })
      .def("view", [](Checkpoint& c, const std::string& name) {
        auto ft = c.get(name);
        return py::make_tuple(tensor_view(ft.first, *ft.second), py::cast(ft.first));
      });

  m.def("hub_cache_root", &hub_cache_root);
  m.def("resolve_model", &resolve_model, py::arg("spec"), py::arg("cache_root") = "");
  m.def("detect_family", [](const std::string& config_json) { return std::string(family_name(detect_family(json::parse(config_json)))); });

  py::enum_<Split>(m, "Split")
      .value("Replicated", Split::Replicated)
      .value("Rows", Split::Rows)
      .value("Cols", Split::Cols)
      .value("Vocab", Split::Vocab)
      .value("Expert", Split::Expert);
  m.def("shard_slice", [](Split split, int world, int rank, int64_t extent, int64_t granule) {
    ShardSpec s;
    s.split = split; s.world = world; s.rank = rank; s.granule = granule;
    const Slice r = shard_slice(s, extent);
    return py::make_tuple(r.begin, r.end);
  }, py::arg("split"), py::arg("world"), py::arg("rank"), py::arg("extent"), py::arg("granule") = 1);
  m.def("expert_slice", [](int experts, int world, int rank) {
    const Slice r = expert_slice(experts, world, rank);
    return py::make_tuple(r.begin, r.end);
  });
}
