// C++ classes with the names, constructor arguments and methods of the reference's public
// template API for the GPU path -- pink::Data, pink::SOM, pink::Trainer<..., float, true>,
// pink::Mapper<..., float, true>, the layouts, enums and neighbourhood functors
// (src/SelfOrganizingMapLib/{Data,SOM,Trainer,Mapper,CartesianLayout,HexagonalLayout}.h,
// src/UtilitiesLib/{DistributionFunctor,Interpolation,DataType,EuclideanDistanceShape}.h) --
// implemented on the C ABI of pink_b200.h.  Header only; link with libpink_b200.so.
//
// Code written against the reference's Trainer / Mapper / SOM / Data compiles against these
// with `UseGPU = true` and `T = float`; the CPU specialisations do not exist here.
#pragma once

#include "pink_b200.h"

#include <array>
#include <cmath>
#include <cstdint>
#include <functional>
#include <numeric>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

namespace pink {

class exception : public std::runtime_error
{
public:
    explicit exception(std::string const& what) : std::runtime_error(what) {}
};

enum class Interpolation { NEAREST_NEIGHBOR, BILINEAR };
enum class DataType { FLOAT, UINT16, UINT8 };
enum class EuclideanDistanceShape { QUADRATIC, CIRCULAR };

namespace detail {
inline void check(int rc) { if (rc != PINK_B200_OK) throw exception(pink_b200_last_error()); }
} // namespace detail

/// n-dimensional cartesian layout; the last two dimensions are (height, width), a leading one the channels
template <uint8_t dim>
struct CartesianLayout
{
    static const uint8_t dimensionality = dim;
    static constexpr const char* type = "CartesianLayout";
    typedef uint32_t IndexType;
    typedef std::array<uint32_t, dim> DimensionType;

    bool operator == (CartesianLayout const& other) const { return m_dimension == other.m_dimension; }
    auto size() const { return std::accumulate(m_dimension.begin(), m_dimension.end(), 1u, std::multiplies<uint32_t>()); }
    auto get_dimension() const { return m_dimension; }
    auto get_dimension(IndexType i) const { return m_dimension[i]; }
    auto get_last_dimension() const { return m_dimension[dim - 1]; }
    /// number of two-dimensional planes an entry consists of
    auto get_spacing() const { return dim == 3 ? m_dimension[0] : 1u; }

    DimensionType m_dimension;
};

/// hexagonal map in axial coordinates stored row by row; both dimensions are the (odd) side length
struct HexagonalLayout
{
    static const uint8_t dimensionality = 2;
    static constexpr const char* type = "HexagonalLayout";
    typedef uint32_t IndexType;
    typedef std::array<uint32_t, 2> DimensionType;

    HexagonalLayout(DimensionType const& dimension) : m_dimension(dimension)
    {
        if (dimension[0] % 2 == 0) throw exception("Only odd dimensions are allowed for hexagonal layout");
        if (dimension[0] != dimension[1]) throw exception("dimension[0] must be identical to dimension[1]");
    }
    bool operator == (HexagonalLayout const& other) const { return m_dimension == other.m_dimension; }
    auto size() const { return pink_b200_som_size(PINK_B200_LAYOUT_HEXAGONAL, m_dimension[0], m_dimension[1]); }
    auto get_dimension() const { return m_dimension; }
    auto get_dimension(IndexType i) const { return m_dimension[i]; }
    auto get_last_dimension() const { return m_dimension[1]; }

    DimensionType m_dimension;
};

namespace detail {
template <typename Layout> struct layout_id;
template <uint8_t dim> struct layout_id<CartesianLayout<dim>> { static constexpr uint32_t value = PINK_B200_LAYOUT_CARTESIAN; };
template <> struct layout_id<HexagonalLayout> { static constexpr uint32_t value = PINK_B200_LAYOUT_HEXAGONAL; };

/// (layout id, dim0, dim1, dim2) of a map layout as the C ABI's per-distance-class functions want it
inline std::array<uint32_t, 4> grid_of(CartesianLayout<1> const& l) { return {PINK_B200_LAYOUT_CARTESIAN, l.m_dimension[0], 1, 1}; }
inline std::array<uint32_t, 4> grid_of(CartesianLayout<2> const& l) { return {PINK_B200_LAYOUT_CARTESIAN, l.m_dimension[0], l.m_dimension[1], 1}; }
inline std::array<uint32_t, 4> grid_of(CartesianLayout<3> const& l)
{ return {PINK_B200_LAYOUT_CARTESIAN, l.m_dimension[0], l.m_dimension[1], l.m_dimension[2]}; }
inline std::array<uint32_t, 4> grid_of(HexagonalLayout const& l) { return {PINK_B200_LAYOUT_HEXAGONAL, l.m_dimension[0], l.m_dimension[1], 1}; }
} // namespace detail

/// one data entry (an image or a neuron)
template <typename Layout, typename T = float>
class Data
{
public:
    typedef T ValueType;
    typedef Layout LayoutType;

    Data() : m_layout{} {}
    explicit Data(Layout const& layout) : m_layout(layout), m_data(layout.size()) {}
    Data(Layout const& layout, T value) : m_layout(layout), m_data(layout.size(), value) {}
    Data(Layout const& layout, std::vector<T> const& data) : m_layout(layout), m_data(data) {}
    Data(Layout const& layout, std::vector<T>&& data) : m_layout(layout), m_data(std::move(data)) {}

    bool operator == (Data const& other) const { return m_layout == other.m_layout && m_data == other.m_data; }
    T& operator [] (uint32_t i) { return m_data[i]; }
    T const& operator [] (uint32_t i) const { return m_data[i]; }
    auto size() const { return m_data.size(); }
    auto get_data_pointer() { return m_data.data(); }
    auto get_data_pointer() const { return m_data.data(); }
    auto get_layout() const { return m_layout; }
    auto get_dimension() const { return m_layout.get_dimension(); }

private:
    Layout m_layout;
    std::vector<T> m_data;
};

/// the map: som_layout.size() neurons of neuron_layout.size() values each
template <typename SOMLayout, typename NeuronLayout, typename T = float>
class SOM
{
public:
    typedef T ValueType;
    typedef SOMLayout SOMLayoutType;
    typedef NeuronLayout NeuronLayoutType;

    SOM(SOMLayout const& som_layout, NeuronLayout const& neuron_layout)
     : m_som_layout(som_layout), m_neuron_layout(neuron_layout), m_data(som_layout.size() * neuron_layout.size()) {}
    SOM(SOMLayout const& som_layout, NeuronLayout const& neuron_layout, T value)
     : m_som_layout(som_layout), m_neuron_layout(neuron_layout), m_data(som_layout.size() * neuron_layout.size(), value) {}
    SOM(SOMLayout const& som_layout, NeuronLayout const& neuron_layout, std::vector<T> const& data)
     : m_som_layout(som_layout), m_neuron_layout(neuron_layout), m_data(data) {}

    bool operator == (SOM const& other) const
    { return m_som_layout == other.m_som_layout && m_neuron_layout == other.m_neuron_layout && m_data == other.m_data; }
    auto size() const { return m_data.size(); }
    auto get_data() const { return m_data; }
    auto get_data_pointer() { return m_data.data(); }
    auto get_data_pointer() const { return m_data.data(); }
    auto get_number_of_neurons() const -> uint32_t { return static_cast<uint32_t>(m_som_layout.size()); }
    auto get_neuron_size() const -> uint32_t { return static_cast<uint32_t>(m_neuron_layout.size()); }
    auto get_som_layout() const { return m_som_layout; }
    auto get_neuron_layout() const { return m_neuron_layout; }
    auto get_som_dimension() const { return m_som_layout.get_dimension(); }
    auto get_neuron_dimension() const { return m_neuron_layout.get_dimension(); }

private:
    SOMLayout m_som_layout;
    NeuronLayout m_neuron_layout;
    std::vector<T> m_data;
};

/// neighbourhood functors (value of the update factor at a map distance)
struct StepFunctor
{
    explicit StepFunctor(float value) : value(value) {}
    float operator () (float distance) const { return distance <= value ? 1.0f : 0.0f; }
    float value;
};

struct GaussianFunctor
{
    GaussianFunctor(float sigma, float damping) : sigma(sigma), damping(damping) {}
    float operator () (float distance) const
    { return damping / (sigma * std::sqrt(2.0f * static_cast<float>(M_PI))) * std::exp(-0.5f * std::pow((distance / sigma), 2.0f)); }
    float sigma, damping;
};

struct UnityGaussianFunctor
{
    UnityGaussianFunctor(float sigma, float damping) : sigma(sigma), damping(damping) {}
    float operator () (float distance) const { return damping * std::exp(-0.5f * std::pow((distance / sigma), 2.0f)); }
    float sigma, damping;
};

struct MexicanHatFunctor
{
    MexicanHatFunctor(float sigma, float damping) : sigma(sigma), damping(damping)
    {
        if (sigma <= 0) throw exception("MexicanHatFunctor: sigma <= 0 not defined.");
    }
    float operator () (float distance) const
    {
        const float sigma2 = sigma * sigma, distance2 = distance * distance;
        return 2.0f * damping / (std::sqrt(3.0f * sigma) * std::pow(static_cast<float>(M_PI), 0.25f))
             * (1.0f - distance2 / sigma2) * std::exp(-distance2 / (2.0f * sigma2));
    }
    float sigma, damping;
};

namespace detail {

/// device state shared by Trainer and Mapper: one context of the C ABI, created with the first image
template <typename SOMLayout, typename DataLayout>
class Session
{
public:
    Session(uint32_t n_neurons, DataLayout const& neuron_layout, uint32_t number_of_rotations, bool use_flip,
        Interpolation interpolation, uint32_t euclidean_distance_dim, EuclideanDistanceShape shape, DataType type)
    {
        if (number_of_rotations == 0 or (number_of_rotations != 1 and number_of_rotations % 4 != 0))
            throw exception("Number of rotations must be 1 or larger then 1 and divisible by 4");
        if (euclidean_distance_dim == 0) throw exception("euclidean_distance_dim not defined");
        m_cfg.n_neurons = n_neurons;
        m_cfg.channels = neuron_layout.get_spacing();
        m_cfg.neuron_dim = neuron_layout.get_last_dimension();
        m_cfg.ed_dim = euclidean_distance_dim;
        m_cfg.ed_shape = shape == EuclideanDistanceShape::QUADRATIC ? PINK_B200_QUADRATIC : PINK_B200_CIRCULAR;
        m_cfg.n_rotations = number_of_rotations;
        m_cfg.use_flip = use_flip;
        m_cfg.dist_type = type == DataType::FLOAT ? PINK_B200_FLOAT : (type == DataType::UINT16 ? PINK_B200_UINT16 : PINK_B200_UINT8);
        m_cfg.interpolation = interpolation == Interpolation::BILINEAR ? PINK_B200_BILINEAR : PINK_B200_NEAREST_NEIGHBOR;
        m_cfg.world_size = 1;
    }
    ~Session() { pink_b200_destroy(m_ctx); }
    Session(Session const&) = delete;
    Session& operator = (Session const&) = delete;

    /// the image size is known with the first image
    pink_b200_ctx* context(Data<DataLayout, float> const& data, float const* som)
    {
        auto&& dim = data.get_dimension();
        if (dim[DataLayout::dimensionality - 1] != dim[DataLayout::dimensionality - 2]) throw exception("Images must be quadratic.");
        if (!m_ctx) {
            m_cfg.image_dim = data.get_layout().get_last_dimension();
            check(pink_b200_create(&m_cfg, &m_ctx));
            check(pink_b200_set_som(m_ctx, som));
        } else if (m_cfg.image_dim != data.get_layout().get_last_dimension()) {
            throw exception("all images of one Trainer or Mapper must have the same size");
        }
        return m_ctx;
    }
    pink_b200_ctx* get() const { return m_ctx; }

private:
    pink_b200_config m_cfg{};
    pink_b200_ctx* m_ctx = nullptr;
};

} // namespace detail

template <typename SOMLayout, typename DataLayout, typename T, bool UseGPU>
class Trainer;

/// GPU trainer: operator() trains one image; the host SOM is refreshed by update_som()
template <typename SOMLayout, typename DataLayout>
class Trainer<SOMLayout, DataLayout, float, true>
{
public:
    typedef SOM<SOMLayout, DataLayout, float> SOMType;

    Trainer(SOMType& som, std::function<float(float)> const& distribution_function, int /*verbosity*/,
        uint32_t number_of_rotations, bool use_flip, float max_update_distance, Interpolation interpolation,
        uint32_t euclidean_distance_dim, EuclideanDistanceShape const& euclidean_distance_shape = EuclideanDistanceShape::QUADRATIC,
        uint32_t /*block_size*/ = 256, DataType euclidean_distance_type = DataType::FLOAT)
     : m_som(som),
       m_session(som.get_number_of_neurons(), som.get_neuron_layout(), number_of_rotations, use_flip, interpolation,
           euclidean_distance_dim, euclidean_distance_shape, euclidean_distance_type),
       m_update_info(som.get_number_of_neurons(), 0)
    {
        // update factor of neuron j when neuron i is the best matching unit: the distribution function of
        // their map distance, cut off at max_update_distance -- evaluated once per distinct distance of the
        // grid (the reference calls it N^2 times, Trainer.h:69-76; the factors are the same)
        m_grid = detail::grid_of(som.get_som_layout());
        const uint32_t classes = pink_b200_distance_classes(m_grid[0], m_grid[1], m_grid[2], m_grid[3], nullptr, 0);
        if (classes == 0) throw exception("unsupported SOM layout");
        std::vector<float> distance(classes);
        pink_b200_distance_classes(m_grid[0], m_grid[1], m_grid[2], m_grid[3], distance.data(), classes);
        m_update_factors.resize(classes);
        for (uint32_t i = 0; i < classes; ++i)
            m_update_factors[i] = (max_update_distance <= 0 or distance[i] < max_update_distance)
                                ? distribution_function(distance[i]) : 0.0f;
    }

    /// Nothing of a training step can be observed before update_som(), so the images are collected and handed to
    /// the device sixteen at a time: whole batches of steps run in one launch.
    void operator () (Data<DataLayout, float> const& data)
    {
        const bool first = m_session.get() == nullptr;
        pink_b200_ctx* ctx = m_session.context(data, m_som.get_data_pointer());
        if (first) detail::check(pink_b200_set_update_lut(ctx, m_grid[0], m_grid[1], m_grid[2], m_grid[3], m_update_factors.data(),
                                                          static_cast<uint32_t>(m_update_factors.size())));
        const float* px = data.get_data_pointer();
        m_pending.insert(m_pending.end(), px, px + data.size());
        if (++m_n_pending == 16) flush();
    }

    /// copy the trained map from the device into the SOM object
    void update_som()
    {
        if (!m_session.get()) return;
        flush();
        detail::check(pink_b200_get_som(m_session.get(), m_som.get_data_pointer()));
        detail::check(pink_b200_get_update_counts(m_session.get(), m_update_info.data()));
    }

    /// how often each neuron was the best matching unit (as of the last update_som())
    auto get_update_info() const { return m_update_info; }

private:
    /// the collected images, in order (the library has taken them out of the buffer when the call returns)
    void flush()
    {
        if (m_n_pending == 0) return;
        const uint32_t n = m_n_pending;
        m_n_pending = 0;
        const int rc = pink_b200_train(m_session.get(), m_pending.data(), n);
        m_pending.clear();
        detail::check(rc);
    }

    SOMType& m_som;
    detail::Session<SOMLayout, DataLayout> m_session;
    std::array<uint32_t, 4> m_grid{};
    std::vector<float> m_pending;               // images given to operator() that have not gone to the device yet
    uint32_t m_n_pending = 0;
    std::vector<float> m_update_factors;        // one factor per distance class of the grid
    std::vector<uint32_t> m_update_info;
};

template <typename SOMLayout, typename DataLayout, typename T, bool UseGPU>
class Mapper;

/// GPU mapper: operator() returns, per neuron, the distance of the image's best transform and its index
template <typename SOMLayout, typename DataLayout>
class Mapper<SOMLayout, DataLayout, float, true>
{
public:
    typedef SOM<SOMLayout, DataLayout, float> SOMType;

    Mapper(SOMType const& som, int /*verbosity*/, uint32_t number_of_rotations, bool use_flip, Interpolation interpolation,
        uint32_t euclidean_distance_dim, EuclideanDistanceShape const& euclidean_distance_shape = EuclideanDistanceShape::QUADRATIC,
        uint32_t /*block_size*/ = 256, DataType euclidean_distance_type = DataType::FLOAT)
     : m_som(som),
       m_session(som.get_number_of_neurons(), som.get_neuron_layout(), number_of_rotations, use_flip, interpolation,
           euclidean_distance_dim, euclidean_distance_shape, euclidean_distance_type)
    {}

    auto operator () (Data<DataLayout, float> const& data)
    {
        pink_b200_ctx* ctx = m_session.context(data, m_som.get_data_pointer());
        std::vector<float> distance(m_som.get_number_of_neurons());
        std::vector<uint32_t> best_transform(m_som.get_number_of_neurons());
        detail::check(pink_b200_map(ctx, data.get_data_pointer(), 1, distance.data(), best_transform.data()));
        return std::make_tuple(distance, best_transform);
    }

private:
    SOMType const& m_som;
    detail::Session<SOMLayout, DataLayout> m_session;
};

} // namespace pink
