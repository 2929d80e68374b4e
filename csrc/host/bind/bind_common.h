// Shared helpers for the pybind11 module: JSON <-> Python object conversion (dict / list /
// str / int / float / bool / None), so every JSON-typed argument or result is a plain
// Python object on the Python side.
#pragma once

#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "core/json.hpp"

namespace py = pybind11;

namespace slime {

inline py::object json_to_py(const Json& j)
{
    switch (j.type()) {
        case Json::Type::Null: return py::none();
        case Json::Type::Bool: return py::bool_(j.as_bool());
        case Json::Type::Int: return py::int_(j.as_int());
        case Json::Type::UInt: return py::int_(j.as_uint());
        case Json::Type::Double: return py::float_(j.as_double());
        case Json::Type::String: return py::str(j.as_string());
        case Json::Type::Array: {
            py::list l;
            for (const auto& v : j.items()) l.append(json_to_py(v));
            return std::move(l);
        }
        case Json::Type::Object: {
            py::dict d;
            for (const auto& kv : j.fields()) d[py::str(kv.first)] = json_to_py(kv.second);
            return std::move(d);
        }
    }
    return py::none();
}

inline Json py_to_json(const py::handle& o)
{
    if (o.is_none()) return Json();
    if (py::isinstance<py::bool_>(o)) return Json(o.cast<bool>());
    if (py::isinstance<py::int_>(o)) {
        // keep full unsigned 64-bit range for addresses
        if (PyObject_RichCompareBool(o.ptr(), py::int_(0).ptr(), Py_LT) == 1) return Json(o.cast<long long>());
        return Json(o.cast<unsigned long long>());
    }
    if (py::isinstance<py::float_>(o)) return Json(o.cast<double>());
    if (py::isinstance<py::str>(o)) return Json(o.cast<std::string>());
    if (py::isinstance<py::bytes>(o)) return Json(o.cast<std::string>());
    if (py::isinstance<py::dict>(o)) {
        Json j = Json::object();
        for (auto item : py::reinterpret_borrow<py::dict>(o)) j[py::str(item.first).cast<std::string>()] = py_to_json(item.second);
        return j;
    }
    if (py::isinstance<py::list>(o) || py::isinstance<py::tuple>(o)) {
        Json j = Json::array();
        for (auto item : o) j.push_back(py_to_json(item));
        return j;
    }
    throw py::type_error("cannot convert object of type " + std::string(py::str(o.get_type())) + " to JSON");
}

}  // namespace slime

namespace pybind11 {
namespace detail {
template<>
struct type_caster<slime::Json> {
public:
    PYBIND11_TYPE_CASTER(slime::Json, const_name("json"));
    bool load(handle src, bool)
    {
        try {
            value = slime::py_to_json(src);
            return true;
        }
        catch (const py::type_error&) {
            return false;
        }
    }
    static handle cast(const slime::Json& src, return_value_policy, handle) { return slime::json_to_py(src).release(); }
};
}  // namespace detail
}  // namespace pybind11
