// ref_cuda_shim.cu -- thin extern "C" window onto the UNMODIFIED reference CUDA implementation
// (Trainer<..., true> / Mapper<..., true>, src/SelfOrganizingMapLib/Trainer.h:198-333, Mapper.h:126-229, and the
// CudaLib kernels behind them), compiled in place from the reference source tree for sm_100a into
// oracle/_ref/libpink_ref_cuda.so by oracle/Makefile.
//
// TEST INFRASTRUCTURE ONLY: a second checker (the reference's own GPU arithmetic) and the "reference on the same
// GPU" line of the benchmark.  The shipped library never links or loads it; no reference source is copied here.
// Use with ONE visible GPU: the reference's multi-GPU branch passes a loop index where a device id is expected
// (src/CudaLib/generate_euclidean_distance_matrix_first_step_multi_gpu.h:95).
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <vector>

#include "SelfOrganizingMapLib/CartesianLayout.h"
#include "SelfOrganizingMapLib/HexagonalLayout.h"
#include "SelfOrganizingMapLib/Data.h"
#include "SelfOrganizingMapLib/SOM.h"
#include "SelfOrganizingMapLib/Trainer.h"
#include "SelfOrganizingMapLib/Mapper.h"
#include "UtilitiesLib/DistributionFunctor.h"

using namespace pink;

namespace {

struct Session
{
    virtual ~Session() {}
    virtual void train(const float* img) = 0;
    virtual void map(const float* img, float* dist, uint32_t* rot) = 0;
    virtual void get_som(float* out) = 0;
};

template <typename SL>
struct SessionT : Session
{
    typedef CartesianLayout<2> DL;
    typedef SOM<SL, DL, float> SOMT;
    SOMT som;
    DL img_layout;
    std::unique_ptr<Trainer<SL, DL, float, true>> trainer;
    std::unique_ptr<Mapper<SL, DL, float, true>> mapper;

    SessionT(SL const& som_layout, const float* som_in, uint32_t id, uint32_t nd, uint32_t ed, uint32_t R, bool flip,
             float sigma, float damping, bool for_map, int dtype)
     : som(som_layout, DL{{nd, nd}}), img_layout(DL{{id, id}})
    {
        std::memcpy(som.get_data_pointer(), som_in, som.size() * sizeof(float));
        const DataType type = dtype == 2 ? DataType::UINT8 : (dtype == 1 ? DataType::UINT16 : DataType::FLOAT);
        if (for_map)
            mapper.reset(new Mapper<SL, DL, float, true>(som, 0, R, flip, Interpolation::BILINEAR, ed,
                                                         EuclideanDistanceShape::QUADRATIC, 256, type));
        else
            trainer.reset(new Trainer<SL, DL, float, true>(som, GaussianFunctor(sigma, damping), 0, R, flip, -1.0f,
                                                           Interpolation::BILINEAR, ed, EuclideanDistanceShape::QUADRATIC,
                                                           256, type));
    }
    void train(const float* img) override
    {
        Data<DL, float> d(img_layout, std::vector<float>(img, img + img_layout.size()));
        (*trainer)(d);
    }
    void map(const float* img, float* dist, uint32_t* rot) override
    {
        Data<DL, float> d(img_layout, std::vector<float>(img, img + img_layout.size()));
        auto r = (*mapper)(d);
        std::memcpy(dist, std::get<0>(r).data(), std::get<0>(r).size() * sizeof(float));
        std::memcpy(rot, std::get<1>(r).data(), std::get<1>(r).size() * sizeof(uint32_t));
    }
    void get_som(float* out) override
    {
        if (trainer) trainer->update_som();
        std::memcpy(out, som.get_data_pointer(), som.size() * sizeof(float));
    }
};

} // namespace

extern "C" {

// som_layout: 0 cartesian-2d (s0 x s1), 1 hexagonal (side s0); single-channel square images of side id;
// dtype: 0 float, 1 uint16, 2 uint8 distances.  Returns NULL when the reference rejects the configuration.
void* ref_cuda_session_create(const float* som, int som_layout, uint32_t s0, uint32_t s1, uint32_t id, uint32_t nd,
                              uint32_t ed, uint32_t R, int flip, float sigma, float damping, int for_map, int dtype)
{
    try {
        if (som_layout == 0)
            return new SessionT<CartesianLayout<2>>(CartesianLayout<2>{{s0, s1}}, som, id, nd, ed, R, flip, sigma, damping, for_map, dtype);
        return new SessionT<HexagonalLayout>(HexagonalLayout({s0, s0}), som, id, nd, ed, R, flip, sigma, damping, for_map, dtype);
    } catch (std::exception const&) {
        return nullptr;
    }
}

void ref_cuda_session_train(void* s, const float* images, uint64_t n, uint64_t image_size)
{
    for (uint64_t i = 0; i < n; ++i) static_cast<Session*>(s)->train(images + i * image_size);
    cudaDeviceSynchronize();
}

void ref_cuda_session_map(void* s, const float* images, uint64_t n, uint64_t image_size, uint64_t N, float* dist, uint32_t* rot)
{
    for (uint64_t i = 0; i < n; ++i) static_cast<Session*>(s)->map(images + i * image_size, dist + i * N, rot + i * N);
}

void ref_cuda_session_get_som(void* s, float* out) { static_cast<Session*>(s)->get_som(out); }
void ref_cuda_session_destroy(void* s) { delete static_cast<Session*>(s); }

} // extern "C"
