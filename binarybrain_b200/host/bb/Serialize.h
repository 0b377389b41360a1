// Binary object format of the reference (include/bb/Object.h:38-58,142-178, include/bb/DataType.h:671-742,
// include/bb/Tensor.h:614-651,2159-2190), so that layers dumped by BinaryBrain load here and the other way round:
//   object  = "BB_OBJ", int64 version (1), uint64 name length, name, object data
//   data    = int64 version of the class, the parent class's data, the members in declaration order
//   bool    = one byte; vector<T> = uint64 count + elements; indices (SaveIndices) = int64 count + int64 each
//   Tensor_<T> data = int64 1, int64 0 (Object base), int64 offset, int64 size, indices shape, indices stride, raw elements
//   Tensor   data = int64 1, int64 0, int32 element type, then the Tensor_<T> data
#pragma once

#include <cstdint>
#include <istream>
#include <sstream>
#include <stdexcept>
#include <ostream>
#include <string>
#include <vector>

#include "Memory.h"

namespace bb {
namespace serial {

template <typename T> inline void Save(std::ostream &os, T const &v) { os.write((char const *)&v, sizeof(T)); }
template <typename T> inline void Load(std::istream &is, T &v)
{
    is.read((char *)&v, sizeof(T));
    if (!is) throw std::runtime_error("LoadObject: unexpected end of data");
}
inline void SaveBool(std::ostream &os, bool v) { std::int8_t b = v ? 1 : 0; Save(os, b); }
inline bool LoadBool(std::istream &is) { std::int8_t b; Load(is, b); return b != 0; }
inline void SaveString(std::ostream &os, std::string const &s)
{
    Save(os, (std::uint64_t)s.size());
    if (!s.empty()) os.write(s.data(), (std::streamsize)s.size());
}
inline std::string LoadString(std::istream &is)
{
    std::uint64_t n; Load(is, n);
    if (n > (1u << 20)) throw std::runtime_error("LoadObject: implausible string length");
    std::string s((std::size_t)n, '\0');
    if (n) is.read(&s[0], (std::streamsize)n);
    return s;
}
// std::vector<index_t> written by SaveValue (uint64 count)
inline void SaveShape(std::ostream &os, indices_t const &v) { Save(os, (std::uint64_t)v.size()); for (auto i : v) Save(os, (std::int64_t)i); }
inline indices_t LoadShape(std::istream &is)
{
    std::uint64_t n; Load(is, n);
    if (n > 64) throw std::runtime_error("LoadObject: implausible rank");
    indices_t v((std::size_t)n);
    for (auto &i : v) { std::int64_t t; Load(is, t); i = (index_t)t; }
    return v;
}
// indices written by SaveIndices (int64 count)
inline void SaveIndices(std::ostream &os, indices_t const &v) { Save(os, (std::int64_t)v.size()); for (auto i : v) Save(os, (std::int64_t)i); }
inline indices_t LoadIndices(std::istream &is)
{
    std::int64_t n; Load(is, n);
    if (n < 0 || n > 64) throw std::runtime_error("LoadObject: implausible rank");
    indices_t v((std::size_t)n);
    for (auto &i : v) { std::int64_t t; Load(is, t); i = (index_t)t; }
    return v;
}

inline void WriteHeader(std::ostream &os, std::string const &name)
{
    os.write("BB_OBJ", 6);
    Save(os, (std::int64_t)1);
    SaveString(os, name);
}
inline void ReadHeader(std::istream &is, std::string const &expect)
{
    char tag[6];
    is.read(tag, 6);
    if (!is || std::string(tag, 6) != "BB_OBJ") throw std::runtime_error("LoadObject: not a BB_OBJ stream");
    std::int64_t ver; Load(is, ver);
    std::string name = LoadString(is);
    if (name != expect) throw std::runtime_error("LoadObject: found " + name + ", expected " + expect);
}
inline void ExpectVersion(std::istream &is, std::int64_t want, char const *what)
{
    std::int64_t v; Load(is, v);
    if (v != want) throw std::runtime_error(std::string("LoadObject: unsupported version of ") + what);
}

// Model::DumpObjectData (include/bb/Model.h:392-420): version 1 and the instance name
inline void SaveModelBase(std::ostream &os, std::string const &name) { Save(os, (std::int64_t)1); SaveString(os, name); }
inline std::string LoadModelBase(std::istream &is)
{
    std::int64_t v; Load(is, v);
    if (v == 0) return std::string();
    if (v != 1) throw std::runtime_error("LoadObject: unsupported version of Model");
    std::int64_t n; Load(is, n);
    if (n < 0 || n > (1 << 20)) throw std::runtime_error("LoadObject: implausible name length");
    std::string s((std::size_t)n, '\0');
    if (n) is.read(&s[0], (std::streamsize)n);
    return s;
}

template <typename T> struct type_name;
template <> struct type_name<float>        { static char const *get() { return "fp32"; }  static constexpr std::int32_t code = BB_TYPE_FP32; };
template <> struct type_name<std::int32_t> { static char const *get() { return "int32"; } static constexpr std::int32_t code = 0x0200 + 32; };

// row-major strides in elements, as the reference's Tensor keeps them
inline indices_t RowMajorStrides(indices_t const &shape)
{
    indices_t s(shape.size());
    index_t k = 1;
    for (std::size_t i = shape.size(); i-- > 0;) { s[i] = k; k *= shape[i]; }
    return s;
}

template <typename T>
inline void SaveTensorData(std::ostream &os, Tensor_<T> const &t)
{
    Save(os, (std::int64_t)1);
    Save(os, (std::int64_t)0);
    Save(os, (std::int64_t)0);                       // offset
    Save(os, (std::int64_t)t.GetSize());
    SaveIndices(os, t.GetShape());
    SaveIndices(os, RowMajorStrides(t.GetShape()));
    os.write((char const *)t.HostConst(), (std::streamsize)(sizeof(T) * (std::size_t)t.GetSize()));
}
template <typename T>
inline void LoadTensorData(std::istream &is, Tensor_<T> &t)
{
    ExpectVersion(is, 1, "Tensor_");
    ExpectVersion(is, 0, "Object");
    std::int64_t offset, size; Load(is, offset); Load(is, size);
    indices_t shape = LoadIndices(is);
    indices_t stride = LoadIndices(is);
    if (offset != 0 || size != CalcShapeSize(shape) || stride != RowMajorStrides(shape)) throw std::runtime_error("LoadObject: tensor view not supported");
    t.Resize(shape);
    is.read((char *)t.Host(true), (std::streamsize)(sizeof(T) * (std::size_t)size));
    if (!is) throw std::runtime_error("LoadObject: unexpected end of data");
}

// typed tensor as its own object ("Tensor_fp32", "Tensor_int32")
template <typename T>
inline void DumpTypedTensor(std::ostream &os, Tensor_<T> const &t) { WriteHeader(os, std::string("Tensor_") + type_name<T>::get()); SaveTensorData(os, t); }
template <typename T>
inline void LoadTypedTensor(std::istream &is, Tensor_<T> &t) { ReadHeader(is, std::string("Tensor_") + type_name<T>::get()); LoadTensorData(is, t); }

// type-erased "Tensor" object holding fp32
inline void DumpTensor(std::ostream &os, Tensor_<float> const &t)
{
    WriteHeader(os, "Tensor");
    Save(os, (std::int64_t)1);
    Save(os, (std::int64_t)0);
    Save(os, (std::int32_t)type_name<float>::code);
    SaveTensorData(os, t);
}
inline void LoadTensor(std::istream &is, Tensor_<float> &t)
{
    ReadHeader(is, "Tensor");
    ExpectVersion(is, 1, "Tensor");
    ExpectVersion(is, 0, "Object");
    std::int32_t code; Load(is, code);
    if (code != type_name<float>::code) throw std::runtime_error("LoadObject: tensor element type is not fp32");
    LoadTensorData(is, t);
}

}   // namespace serial
}   // namespace bb
