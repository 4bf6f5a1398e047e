// TEST INFRASTRUCTURE ONLY.  Stand-in for LibAPR's ParticleData<T> / VectorData<T> as used by the
// reference's CPU operators (helpers.hpp:166,194; conv.hpp:109,316-322,338-339).
//
// `data.resize(n, v)` assigns `v` to ALL n elements.  The reference's backward pass declares one
// tree buffer outside its input-channel loop (conv.hpp:317) and relies on
// `tree_data.data.resize(n, 0)` (helpers.hpp:166) to hand fill_tree_mean a zeroed tree for every
// channel; its forward pass creates a fresh object per channel (conv.hpp:109).  Plain
// std::vector::resize would keep the previous channel's sums.
#ifndef ORACLE_SHIM_PARTICLEDATA_HPP
#define ORACLE_SHIM_PARTICLEDATA_HPP

#include <cstdint>
#include <vector>
#include <algorithm>

template<typename T>
class VectorData {
public:
    std::vector<T> vec;
    void resize(uint64_t n) { vec.resize(n); }
    void resize(uint64_t n, T v) { vec.assign(n, v); }
    uint64_t size() const { return vec.size(); }
    T& operator[](uint64_t i) { return vec[i]; }
    const T& operator[](uint64_t i) const { return vec[i]; }
    typename std::vector<T>::iterator begin() { return vec.begin(); }
    typename std::vector<T>::iterator end() { return vec.end(); }
};

template<typename T>
class ParticleData {
public:
    VectorData<T> data;
    ParticleData() = default;
    explicit ParticleData(uint64_t n) { data.resize(n, T(0)); }
    void init(uint64_t n) { data.resize(n, T(0)); }
    uint64_t size() const { return data.size(); }
    T& operator[](uint64_t i) { return data.vec[i]; }
    const T& operator[](uint64_t i) const { return data.vec[i]; }
    typename std::vector<T>::iterator begin() { return data.vec.begin(); }
    typename std::vector<T>::iterator end() { return data.vec.end(); }
    void set_to_zero() { std::fill(data.vec.begin(), data.vec.end(), T(0)); }
};

#endif
