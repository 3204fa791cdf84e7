// pyngp_module.cpp -- the `pyngp` Python module of the reference (internal/python_api.cu:43-134), compiled against the
// C++ host of this library (include/srf_testbed.hpp) instead of the reference's Testbed.  A driver written for the
// reference (`import pyngp as ngp`; experiment/*/python/run.py) runs its inference half unchanged with
// `from sphericalrf_b200 import pyngp as ngp`.  All host logic is C++ (configuration and snapshot parsing, camera
// conventions, the spp loop); the arithmetic happens in libsrf_b200.so on the GPU.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <array>

#include "srf_testbed.hpp"

namespace py = pybind11;
using srf_host::Json;
using srf_host::RenderingBuffer;
using srf_host::Testbed;

namespace {

// The five enums of the reference's module, with its member names and order.
enum class Activation : int { None = 0, ReLU, Logistic, Exponential };
enum class RenderMode : int { AO = 0, Shade, Normals, Depth, Distance, Cost };
enum class ColorSpace : int { Linear = 0, SRGB, VisPosNeg };
enum class TonemapCurve : int { Identity = 0, ACES, Hable, Reinhard };
enum class LossType : int { L2 = 0, L1, Mape, Smape, SmoothL1, LogL1, RelativeL2 };

// A Python object (dict / list / str / number / bool / None / bytes) as a Json document.
Json json_from_python(const py::handle& o) {
    if (o.is_none()) return Json();
    if (py::isinstance<py::bool_>(o)) return Json::boolean(o.cast<bool>());
    if (py::isinstance<py::int_>(o)) return Json::integer(o.cast<int64_t>());
    if (py::isinstance<py::float_>(o)) return Json::number(o.cast<double>());
    if (py::isinstance<py::str>(o)) return Json::string(o.cast<std::string>());
    if (py::isinstance<py::bytes>(o)) return Json::binary(o.cast<std::string>());
    if (py::isinstance<py::dict>(o)) {
        Json j = Json::object();
        for (auto kv : py::reinterpret_borrow<py::dict>(o)) j.set(py::str(kv.first).cast<std::string>(), json_from_python(kv.second));
        return j;
    }
    if (py::isinstance<py::list>(o) || py::isinstance<py::tuple>(o)) {
        Json j = Json::array();
        for (auto item : py::reinterpret_borrow<py::sequence>(o)) j.push_back(json_from_python(item));
        return j;
    }
    throw std::runtime_error("model configuration holds a value that is not JSON");
}

py::object python_from_json(const Json& j) {
    switch (j.type()) {
    case Json::Null: return py::none();
    case Json::Bool: return py::bool_(j.as_bool());
    case Json::Int: return py::int_(j.as_int());
    case Json::Float: return py::float_(j.as_double());
    case Json::String: return py::str(j.as_string());
    case Json::Binary: return py::bytes(j.as_string());
    case Json::Array: { py::list l; for (size_t i = 0; i < j.size(); ++i) l.append(python_from_json(j.at(i))); return std::move(l); }
    case Json::Object: { py::dict d; for (const auto& kv : j.members()) d[py::str(kv.first)] = python_from_json(kv.second); return std::move(d); }
    }
    return py::none();
}

using Cam = py::array_t<float, py::array::c_style | py::array::forcecast>;

}  // namespace

PYBIND11_MODULE(pyngp, m) {
    m.doc() = "SphericalRF render path on B200: the reference's pyngp surface over libsrf_b200.so";

    py::enum_<Activation>(m, "Activation")
        .value("None", Activation::None).value("ReLU", Activation::ReLU).value("Logistic", Activation::Logistic)
        .value("Exponential", Activation::Exponential).export_values();
    py::enum_<RenderMode>(m, "RenderMode")
        .value("AO", RenderMode::AO).value("Shade", RenderMode::Shade).value("Normals", RenderMode::Normals)
        .value("Depth", RenderMode::Depth).value("Distance", RenderMode::Distance).value("Cost", RenderMode::Cost).export_values();
    py::enum_<ColorSpace>(m, "ColorSpace")
        .value("Linear", ColorSpace::Linear).value("SRGB", ColorSpace::SRGB).export_values();
    py::enum_<TonemapCurve>(m, "TonemapCurve")
        .value("Identity", TonemapCurve::Identity).value("ACES", TonemapCurve::ACES).value("Hable", TonemapCurve::Hable)
        .value("Reinhard", TonemapCurve::Reinhard).export_values();
    py::enum_<LossType>(m, "LossType")
        .value("L2", LossType::L2).value("L1", LossType::L1).value("Mape", LossType::Mape).value("Smape", LossType::Smape)
        .value("SmoothL1", LossType::SmoothL1).value("LogL1", LossType::LogL1).value("RelativeL2", LossType::RelativeL2).export_values();

    py::class_<Testbed> testbed(m, "Testbed");
    testbed
        .def(py::init([]() { return new Testbed(0); }))
        .def(py::init([](int device) { return new Testbed(device); }), py::arg("device"))
        // Configuration & I/O
        .def("load_model_config", &Testbed::load_model_config, "Reload the network from a config file.")
        .def("load_model_config_dict", [](Testbed& t, const py::dict& d) { t.load_model_config_json(json_from_python(d)); },
             "The same from an already parsed configuration.")
        .def("save_snapshot", [](Testbed& t, const std::string& p, bool o) { t.save_snapshot(p, o); }, py::arg("snapshot_path"),
             py::arg("serialize_optimizer") = false, "Not part of this library: raises.")
        .def("load_snapshot", &Testbed::load_snapshot, py::arg("snapshot_path"), "Load a previously saved snapshot")
        .def("load_training_data", [](Testbed& t, py::args, py::kwargs) { t.load_training_data(""); }, "Not part of this library: raises.")
        .def("load_parameters",
             [](Testbed& t, py::array_t<uint16_t, py::array::c_style> table, py::array_t<uint16_t, py::array::c_style> dmlp,
                py::array_t<uint16_t, py::array::c_style> rmlp, py::array_t<float, py::array::c_style | py::array::forcecast> grid,
                float scene_scale, std::array<float, 3> scene_offset) {
                 if ((size_t)dmlp.size() != srf_host::kDensityMlpParams || (size_t)rmlp.size() != srf_host::kRgbMlpParams)
                     throw std::runtime_error("density MLP must hold 3072 and colour MLP 7168 fp16 parameters");
                 t.load_parameters(table.data(), (size_t)table.size(), dmlp.data(), rmlp.data(), grid.data(), (size_t)grid.size());
                 t.m_scene_scale = scene_scale;
                 for (int i = 0; i < 3; ++i) t.m_scene_offset[i] = scene_offset[i];
             },
             py::arg("hash_table"), py::arg("density_mlp"), py::arg("rgb_mlp"), py::arg("density_grid"), py::arg("scene_scale") = 1.0f,
             py::arg("scene_offset") = std::array<float, 3>{0.5f, 0.5f, 0.5f},
             "What load_snapshot restores, from arrays (fp16 parameters as uint16 bit patterns).")
        // Training
        .def("train", [](Testbed& t, py::args, py::kwargs) { t.train(0, 0); }, "Not part of this library: raises.")
        // Rendering
        .def("render",
             [](Testbed& t, int width, int height, int spp, bool to_srgb) {
                 py::array_t<float> image({height, width, 4});
                 float* p = image.mutable_data();
                 {
                     py::gil_scoped_release release;
                     t.render(width, height, spp, to_srgb, p);
                 }
                 return image;
             },
             "Renders an image at the requested resolution.", py::arg("width") = 1920, py::arg("height") = 1080, py::arg("spp") = 1,
             py::arg("to_srgb") = true)
        // Interesting members
        .def_property("loss_type", [](const Testbed& t) { return (LossType)t.m_loss_type; }, [](Testbed& t, LossType v) { t.m_loss_type = (int)v; })
        .def_property("density_activation", [](const Testbed& t) { return (Activation)t.m_density_activation; },
                      [](Testbed& t, Activation v) { t.m_density_activation = (int)v; })
        .def_property("rgb_activation", [](const Testbed& t) { return (Activation)t.m_rgb_activation; },
                      [](Testbed& t, Activation v) { t.m_rgb_activation = (int)v; })
        .def_property("background_color",
                      [](const Testbed& t) { return std::array<float, 4>{t.m_background_color[0], t.m_background_color[1], t.m_background_color[2], t.m_background_color[3]}; },
                      [](Testbed& t, const std::array<float, 4>& c) { for (int i = 0; i < 4; ++i) t.m_background_color[i] = c[i]; })
        .def_property("color_space", [](const Testbed& t) { return (ColorSpace)t.m_color_space; }, [](Testbed& t, ColorSpace v) { t.m_color_space = (int)v; })
        .def_property_readonly("training_buffer", [](const Testbed&) -> py::object { throw std::runtime_error("training is not part of this library: no training buffer"); })
        .def_property_readonly("rendering_buffer", [](Testbed& t) -> RenderingBuffer& { return t.m_rendering_buffer; }, py::return_value_policy::reference_internal)
        .def_property("fov", &Testbed::fov, &Testbed::set_fov)
        .def_property("fov_xy", [](const Testbed& t) { float o[2]; t.fov_xy(o); return std::array<float, 2>{o[0], o[1]}; },
                      [](Testbed& t, const std::array<float, 2>& v) { t.set_fov_xy(v.data()); })
        .def("set_nerf_camera_matrix",
             [](Testbed& t, Cam cam) {
                 if (cam.size() != 12) throw std::runtime_error("the camera matrix is 3 x 4");
                 t.set_nerf_camera_matrix(cam.data());
             })
        // members of this library (no counterpart in the reference's module)
        .def_property("scene_scale", [](const Testbed& t) { return t.m_scene_scale; }, [](Testbed& t, float v) { t.m_scene_scale = v; })
        .def_property("scene_offset", [](const Testbed& t) { return std::array<float, 3>{t.m_scene_offset[0], t.m_scene_offset[1], t.m_scene_offset[2]}; },
                      [](Testbed& t, const std::array<float, 3>& v) { for (int i = 0; i < 3; ++i) t.m_scene_offset[i] = v[i]; })
        .def_property_readonly("camera_matrix", [](const Testbed& t) {
            py::array_t<float> a({3, 4});
            memcpy(a.mutable_data(), t.m_rendering_buffer.camera_matrix, 12 * sizeof(float));
            return a;
        }, "the camera after set_nerf_camera_matrix's conversion (row-major 3 x 4)")
        .def_property_readonly("model_config", [](const Testbed& t) { return python_from_json(t.model_config()); })
        .def_property_readonly("context", [](Testbed& t) { return (uintptr_t)t.context(); }, "the srf_ctx* of the C-ABI, as an integer")
        .def("train_prep_nerf", &Testbed::train_prep_nerf, py::arg("training_step") = 0u, "One density-grid refresh.");

    py::class_<RenderingBuffer>(testbed, "RenderingBuffer")
        .def_property("render_mode", [](const RenderingBuffer& b) { return (RenderMode)b.render_mode; }, [](RenderingBuffer& b, RenderMode v) { b.render_mode = (int)v; })
        .def_property("tonemap_curve", [](const RenderingBuffer& b) { return (TonemapCurve)b.tonemap_curve; },
                      [](RenderingBuffer& b, TonemapCurve v) { b.tonemap_curve = (int)v; })
        .def_readwrite("exposure", &RenderingBuffer::exposure)
        .def_readwrite("fov_axis", &RenderingBuffer::fov_axis)
        .def_property("relative_focal_length", [](const RenderingBuffer& b) { return std::array<float, 2>{b.relative_focal_length[0], b.relative_focal_length[1]}; },
                      [](RenderingBuffer& b, const std::array<float, 2>& v) { b.relative_focal_length[0] = v[0]; b.relative_focal_length[1] = v[1]; })
        .def_property("principal_point", [](const RenderingBuffer& b) { return std::array<float, 2>{b.principal_point[0], b.principal_point[1]}; },
                      [](RenderingBuffer& b, const std::array<float, 2>& v) { b.principal_point[0] = v[0]; b.principal_point[1] = v[1]; })
        .def_readwrite("MIN_STEPS_INBETWEEN_COMPACTION", &RenderingBuffer::MIN_STEPS_INBETWEEN_COMPACTION)
        .def_readwrite("MAX_STEPS_INBETWEEN_COMPACTION", &RenderingBuffer::MAX_STEPS_INBETWEEN_COMPACTION);

    // host-logic taps for the tests: the C++ parsers on Python data
    m.def("parse_config", [](const py::dict& d) {
        const srf_config_t c = srf_host::parse_config(json_from_python(d));
        return py::bytes((const char*)&c, sizeof(c));
    }, "srf_config_t (as bytes) the C++ host derives from a configuration dictionary");
    m.def("parse_json", [](const std::string& text) { return python_from_json(srf_host::JsonTextParser(text).parse()); },
          "the C++ JSON reader (comments allowed)");
    m.def("parse_msgpack", [](const py::bytes& b) {
        const std::string s = b;
        return python_from_json(srf_host::MsgpackReader((const unsigned char*)s.data(), s.size()).parse());
    }, "the C++ msgpack reader");
    m.def("write_msgpack", [](const py::object& o) { std::string out; srf_host::msgpack_write(json_from_python(o), out); return py::bytes(out); },
          "the C++ msgpack writer");
}
