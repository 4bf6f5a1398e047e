// TEST INFRASTRUCTURE ONLY — never linked into the product library.
//
// Minimal stand-in for the part of LibAPR's `APR` / `LinearIterator` interface that the
// reference's CPU operators call (pyapr/aprnet/src/helpers.hpp, conv.hpp, maxpool.hpp,
// upsample.hpp).  LibAPR itself is an un-vendored submodule of the reference
// (.gitmodules: external/LibAPR) and is not available, so the iterator semantics below restate
// what the call sites require:
//   * begin(level, z, x) positions the iterator on the first particle of that sparse row and
//     returns its global index; end() is one past the row's last particle
//     (helpers.hpp:187,213; conv333_gpu.cu:65-67 for the row addressing);
//   * the iterator converts implicitly to its current global index (helpers.hpp:194,220);
//   * y() is the y coordinate of the current particle (helpers.hpp:189);
//   * particles_level_begin/end(level) bound a level's contiguous index range and
//     total_number_particles(level) is the cumulative count up to and including `level`
//     (helpers.hpp:93-97,166).
// Storage is this project's own CSR form: rows numbered level-major, then z, then x.
#ifndef ORACLE_SHIM_APR_HPP
#define ORACLE_SHIM_APR_HPP

#include <cstdint>
#include <vector>
#include <cmath>
#include <algorithm>

struct ShimAccess {
    int level_min = 0, level_max = 0;
    std::vector<int> z_num, x_num, y_num;      // indexed by level (0..level_max)
    std::vector<int64_t> row_off;              // first row number of each level (size level_max + 2)
    std::vector<int64_t> row_ptr;              // CSR over rows
    std::vector<uint16_t> y_vec;

    void init(int lmin, int lmax, const std::vector<int>& zn, const std::vector<int>& xn,
              const std::vector<int>& yn) {
        level_min = lmin; level_max = lmax; z_num = zn; x_num = xn; y_num = yn;
        row_off.assign(lmax + 2, 0);
        for (int l = 0; l <= lmax; ++l) {
            int64_t rows = (l >= lmin) ? int64_t(z_num[l]) * x_num[l] : 0;
            row_off[l + 1] = row_off[l] + rows;
        }
    }
};

class LinearIterator {
public:
    const ShimAccess* acc = nullptr;
    uint64_t current_index = 0, end_index = 0;

    LinearIterator() = default;
    explicit LinearIterator(const ShimAccess* a) : acc(a) {}

    inline uint64_t begin(const int level, const int z, const int x) {
        const int64_t r = acc->row_off[level] + int64_t(z) * acc->x_num[level] + x;
        current_index = uint64_t(acc->row_ptr[r]);
        end_index = uint64_t(acc->row_ptr[r + 1]);
        return current_index;
    }
    inline uint64_t end() const { return end_index; }
    inline operator uint64_t() const { return current_index; }
    inline LinearIterator& operator++() { ++current_index; return *this; }
    inline LinearIterator operator++(int) { LinearIterator t(*this); ++current_index; return t; }
    inline int y() const { return acc->y_vec[current_index]; }

    inline int x_num(int level) const { return acc->x_num[level]; }
    inline int y_num(int level) const { return acc->y_num[level]; }
    inline int z_num(int level) const { return acc->z_num[level]; }
    inline int level_min() const { return acc->level_min; }
    inline int level_max() const { return acc->level_max; }

    inline uint64_t particles_level_begin(int level) const { return uint64_t(acc->row_ptr[acc->row_off[level]]); }
    inline uint64_t particles_level_end(int level) const { return uint64_t(acc->row_ptr[acc->row_off[level + 1]]); }
    inline uint64_t total_number_particles(int level) const { return particles_level_end(level); }
    inline uint64_t total_number_particles() const { return acc->y_vec.size(); }
    inline uint64_t level_size(int level) const { return uint64_t(1) << level; }
};

class APR {
public:
    ShimAccess parts, tree;
    int dims_yxz[3] = {0, 0, 0};

    LinearIterator iterator() { return LinearIterator(&parts); }
    LinearIterator tree_iterator() { return LinearIterator(&tree); }
    int level_max() const { return parts.level_max; }
    int level_min() const { return parts.level_min; }
    int org_dims(int d) const { return dims_yxz[d]; }
    uint64_t total_number_particles() const { return parts.y_vec.size(); }
    uint64_t total_number_tree_particles() const { return tree.y_vec.size(); }
};

#endif
