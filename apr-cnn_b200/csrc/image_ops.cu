// Particle features <-> dense image at the resolution of level cml = level_max - level_delta.
//
//   reconstruct:       image[c][z][x][y] = value of the particle (or upgraded tree node) whose cell covers
//                      the voxel (piecewise-constant reconstruction); adjoint: sum of the image over the cell
//   sample_particles:  particle = mean of the image over its cell (cells are clipped at the volume border,
//                      the divisor is the clipped volume); adjoint: every voxel of the cell gets value / volume
//
// Arithmetic follows pyapr/aprnet/cuda/src/reconstruct_gpu.cu:5-157 and sample_particles_gpu.cu:5-170.  The
// reference launches one block per (image row, level) and combines the rows of a coarse cell with
// atomicAdd; here a particle is owned by one thread (cells of one voxel) or one warp (larger cells, lanes
// sweep the cell with y fastest and are combined by shuffles in a fixed order), so every result has one
// writer and the sums are deterministic.
#include "apr_device.cuh"

namespace {

typedef long long ll;
constexpr int TPB = 256;

template<typename T> struct DT;
template<> struct DT<float> { static constexpr int id = APRNET_F32; };
template<> struct DT<double> { static constexpr int id = APRNET_F64; };

struct ImageLevel {
    const ll* row_ptr;      // CSR row pointers of the structure this level is read from (particles or tree)
    const uint16_t* y;
    ll row_off;             // first row of the level
    int x_num, k;           // rows per z at this level; cell edge = 2^k voxels
    ll index_offset;        // feature index = structure index + index_offset (upgraded tree nodes)
    int Z, X, Y;            // image extents
};

// to_image: image <- particle value (* 1/volume when `mean`);  else: particle <- sum (or mean) of the image
template<typename T, bool TO_IMAGE>
__global__ void __launch_bounds__(TPB) cell_transfer_kernel(ImageLevel L, T* __restrict__ parts, ll ld, T* __restrict__ image, int C, int mean) {
    const ll r = blockIdx.x;
    const ll pb = L.row_ptr[L.row_off + r], pe = L.row_ptr[L.row_off + r + 1];
    if (pe <= pb) return;
    const int s = 1 << L.k;
    const int z0 = (int) (r / L.x_num) * s, x0 = (int) (r % L.x_num) * s;
    const int z1 = min(z0 + s, L.Z), x1 = min(x0 + s, L.X);
    const ll plane = (ll) L.X * L.Y, vol_img = (ll) L.Z * plane;
    if (L.k == 0) {
        for (ll p = pb + threadIdx.x; p < pe; p += TPB) {
            const ll v = (ll) z0 * plane + (ll) x0 * L.Y + L.y[p];
            for (int c = 0; c < C; ++c) {
                if (TO_IMAGE) image[c * vol_img + v] = parts[c * ld + p + L.index_offset];
                else parts[c * ld + p + L.index_offset] = image[c * vol_img + v];
            }
        }
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (ll p = pb + warp; p < pe; p += TPB / 32) {
        const int y0 = (int) L.y[p] * s, y1 = min(y0 + s, L.Y);
        const int ny = y1 - y0, nx = x1 - x0;
        const ll cells = (ll) (z1 - z0) * nx * ny;
        const T inv = mean ? T(1) / (T) cells : T(1);
        for (int c = 0; c < C; ++c) {
            T* img = image + c * vol_img;
            if (TO_IMAGE) {
                const T v = parts[c * ld + p + L.index_offset] * inv;
                for (ll e = lane; e < cells; e += 32) {
                    const int dy = (int) (e % ny), dx = (int) ((e / ny) % nx), dz = (int) (e / ((ll) ny * nx));
                    img[(ll) (z0 + dz) * plane + (ll) (x0 + dx) * L.Y + y0 + dy] = v;
                }
            } else {
                T acc = 0;
                for (ll e = lane; e < cells; e += 32) {
                    const int dy = (int) (e % ny), dx = (int) ((e / ny) % nx), dz = (int) (e / ((ll) ny * nx));
                    acc += img[(ll) (z0 + dz) * plane + (ll) (x0 + dx) * L.Y + y0 + dy];
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
                if (lane == 0) parts[c * ld + p + L.index_offset] = acc * inv;
            }
        }
    }
}

template<typename T, bool TO_IMAGE>
int run_levels(const aprnet_apr* a, int dl, int C, T* parts, ll ld, T* image, int mean, cudaStream_t st) {
    const int cml = a->cml(dl);
    const LevelMeta& m = a->meta;
    ImageLevel L;
    L.Z = m.z_num[cml]; L.X = m.x_num[cml]; L.Y = m.y_num[cml];
    const char* pname = TO_IMAGE ? "cells_to_image" : "image_to_cells";
    for (int l = m.level_min; l <= cml; ++l) {
        const ll rows = (ll) m.z_num[l] * m.x_num[l];
        if (rows == 0 || m.lvl_begin[l + 1] == m.lvl_begin[l]) continue;
        L.row_ptr = a->row_ptr; L.y = a->y; L.row_off = m.row_off[l]; L.x_num = m.x_num[l]; L.k = cml - l; L.index_offset = 0;
        { AprnetProfScope _prof(pname, st);
        cell_transfer_kernel<T, TO_IMAGE><<<(unsigned) rows, TPB, 0, st>>>(L, parts, ld, image, C, mean);
        }
    }
    if (dl > 0) {      // upgraded tree nodes of level cml, stored behind the particles
        const ll rows = (ll) m.z_num[cml] * m.x_num[cml];
        L.row_ptr = a->tree_row_ptr; L.y = a->tree_y; L.row_off = m.trow_off[cml]; L.x_num = m.x_num[cml]; L.k = 0;
        L.index_offset = a->tree_offset(cml);
        if (rows > 0) {
            AprnetProfScope _prof(pname, st);
            cell_transfer_kernel<T, TO_IMAGE><<<(unsigned) rows, TPB, 0, st>>>(L, parts, ld, image, C, mean);
        }
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<bool TO_IMAGE>
int dispatch(const aprnet_apr* a, int dl, int dtype, int C, void* parts, ll ld, void* image, int mean, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && C > 0 && parts && image, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld >= a->number_parts(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    if (dtype == APRNET_F32) return run_levels<float, TO_IMAGE>(a, dl, C, (float*) parts, ld, (float*) image, mean, st);
    if (dtype == APRNET_F64) return run_levels<double, TO_IMAGE>(a, dl, C, (double*) parts, ld, (double*) image, mean, st);
    aprnet_set_error("unsupported dtype %d", dtype);
    return APRNET_ERR_ARG;
}

} // namespace

extern "C" int aprnet_image_dims(const aprnet_apr* a, int dl, int* z, int* x, int* y) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && z && x && y, "bad argument");
    const int cml = a->cml(dl);
    *z = a->meta.z_num[cml]; *x = a->meta.x_num[cml]; *y = a->meta.y_num[cml];
    return APRNET_OK;
}

// image (C, Z, X, Y) of aprnet_image_dims(); every voxel is written (the cells tile the volume)
extern "C" int aprnet_reconstruct_forward(const aprnet_apr* a, int dl, int dtype, int C, const void* input, int64_t ld_in, void* image, void* stream) {
    return dispatch<true>(a, dl, dtype, C, const_cast<void*>(input), ld_in, image, 0, stream);
}
extern "C" int aprnet_reconstruct_backward(const aprnet_apr* a, int dl, int dtype, int C, const void* grad_image, void* grad_input, int64_t ld_in, void* stream) {
    return dispatch<false>(a, dl, dtype, C, grad_input, ld_in, const_cast<void*>(grad_image), 0, stream);
}
extern "C" int aprnet_sample_particles_forward(const aprnet_apr* a, int dl, int dtype, int C, const void* image, void* output, int64_t ld_out, void* stream) {
    return dispatch<false>(a, dl, dtype, C, output, ld_out, const_cast<void*>(image), 1, stream);
}
extern "C" int aprnet_sample_particles_backward(const aprnet_apr* a, int dl, int dtype, int C, const void* grad_output, int64_t ld_out, void* grad_image, void* stream) {
    return dispatch<true>(a, dl, dtype, C, const_cast<void*>(grad_output), ld_out, grad_image, 1, stream);
}
