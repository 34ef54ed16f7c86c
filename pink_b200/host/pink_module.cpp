// Compiled Python module `_pink`: the reference's pybind11 interface (src/pink/pink.cpp:25-153 -- Data, SOM,
// Trainer, Mapper, GaussianFunctor, the enums, __version__) on the C ABI of this library.  Same class names,
// constructor keywords, defaults, return types and exception texts; Data and SOM expose their storage through
// the buffer protocol like the reference's DynamicData / DynamicSOM (src/pink/DynamicSOM.cpp:15-62), so
// numpy.array(som, copy=False) sees the weights Trainer.update_som() wrote.  use_gpu = False is refused: there
// is no CPU implementation behind this module.  Trainer.train / Mapper.map (many images per call) and
// Trainer.get_update_info are additions.
#include "../../include/pink_b200.h"

#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

// the reference's pink::exception is a std::runtime_error; pybind11 turns it into RuntimeError
struct pink_error : std::runtime_error { using std::runtime_error::runtime_error; };

void check(int rc)
{
    if (rc != PINK_B200_OK) throw pink_error(pink_b200_last_error());
}

enum class Interpolation { NEAREST_NEIGHBOR, BILINEAR };
enum class DataType { FLOAT, UINT16, UINT8 };
enum class Layout { CARTESIAN, HEXAGONAL };
enum class EuclideanDistanceShape { QUADRATIC, CIRCULAR };

// src/UtilitiesLib/DistributionFunctor.cpp:24-33, float arithmetic
struct GaussianFunctor
{
    GaussianFunctor(float sigma, float damping) : sigma(sigma), damping(damping) {}
    float operator()(float distance) const
    {
        return damping / (sigma * std::sqrt(2.0f * static_cast<float>(M_PI))) * std::exp(-0.5f * std::pow((distance / sigma), 2.0f));
    }
    float sigma, damping;
};

std::vector<float> copy_float_buffer(const py::buffer& b, const std::string& data_type, std::vector<uint32_t>* shape)
{
    if (data_type != "float32") throw pink_error("data-type not supported");
    py::buffer_info info = b.request();
    if (info.format != py::format_descriptor<float>::format()) throw pink_error("data-type not supported");
    shape->assign(info.shape.begin(), info.shape.end());
    size_t n = 1;
    for (auto s : info.shape) n *= (size_t)s;
    // the reference copies the buffer too; it must be C-contiguous
    ssize_t expect = sizeof(float);
    for (ssize_t d = info.ndim - 1; d >= 0; --d) {
        if (info.shape[d] > 1 && info.strides[d] != expect) throw pink_error("buffer must be C-contiguous");
        expect *= info.shape[d];
    }
    std::vector<float> out(n);
    std::memcpy(out.data(), info.ptr, n * sizeof(float));
    return out;
}

py::buffer_info float_buffer_info(std::vector<float>& data, const std::vector<uint32_t>& shape)
{
    std::vector<ssize_t> shp(shape.begin(), shape.end()), strides(shape.size());
    ssize_t s = sizeof(float);
    for (ssize_t d = (ssize_t)shape.size() - 1; d >= 0; --d) { strides[d] = s; s *= shp[d]; }
    return py::buffer_info(data.data(), sizeof(float), py::format_descriptor<float>::format(), (ssize_t)shape.size(), shp, strides);
}

struct Data
{
    Data(const py::buffer& b, const std::string& data_type, const std::string& layout) : layout(layout)
    {
        data = copy_float_buffer(b, data_type, &shape);
        const std::map<std::string, size_t> dims = {{"cartesian-1d", 1}, {"cartesian-2d", 2}, {"cartesian-3d", 3}};
        auto it = dims.find(layout);
        if (it == dims.end()) throw pink_error("layout " + layout + " is not supported");
        if (shape.size() != it->second) throw pink_error("layout " + layout + " does not match the buffer's dimensions");
    }
    std::string layout;
    std::vector<uint32_t> shape;
    std::vector<float> data;
};

struct SOM
{
    SOM(const py::buffer& b, const std::string& data_type, const std::string& som_layout_, const std::string& neuron_layout_)
     : som_layout(som_layout_), neuron_layout(neuron_layout_)
    {
        data = copy_float_buffer(b, data_type, &shape);
        const std::map<std::string, size_t> dims = {{"cartesian-1d", 1}, {"cartesian-2d", 2}, {"cartesian-3d", 3}};
        auto it = dims.find(neuron_layout);
        if (it == dims.end()) throw pink_error("neuron layout " + neuron_layout + " is not supported");
        const size_t nn = it->second;
        if (som_layout == "cartesian-2d") {
            if (shape.size() != 2 + nn) throw pink_error("SOM buffer must have shape (som_w, som_h, neuron...)");
            layout = PINK_B200_LAYOUT_CARTESIAN; dim0 = shape[0]; dim1 = shape[1];
            neuron_shape.assign(shape.begin() + 2, shape.end());
        } else if (som_layout == "hexagonal-2d") {
            if (shape.size() != 1 + nn) throw pink_error("hexagonal SOM buffer must have shape (number_of_neurons, neuron...)");
            const uint32_t dim = (uint32_t)std::sqrt((double)((4 * (uint64_t)shape[0] - 1) / 3));      // HexagonalLayout::get_dim_from_size
            if (pink_b200_som_size(PINK_B200_LAYOUT_HEXAGONAL, dim, dim) != shape[0])
                throw pink_error(std::to_string(shape[0]) + " is not the size of a hexagonal SOM");
            layout = PINK_B200_LAYOUT_HEXAGONAL; dim0 = dim1 = dim;
            neuron_shape.assign(shape.begin() + 1, shape.end());
        } else {
            throw pink_error("SOM layout " + som_layout + " is not supported");
        }
        n_neurons = pink_b200_som_size(layout, dim0, dim1);
    }
    // channels and side of a neuron as the library wants them
    void neuron_geometry(uint32_t* channels, uint32_t* side) const
    {
        if (neuron_layout == "cartesian-1d") throw pink_error("Not implemented yet.");       // generate_rotated_images.h:37-47
        uint32_t c = 1, h, w;
        if (neuron_layout == "cartesian-2d") { h = neuron_shape[0]; w = neuron_shape[1]; }
        else { c = neuron_shape[0]; h = neuron_shape[1]; w = neuron_shape[2]; }
        if (h != w) throw pink_error("neurons must be quadratic");
        *channels = c; *side = h;
    }
    std::string som_layout, neuron_layout;
    std::vector<uint32_t> shape, neuron_shape;
    std::vector<float> data;
    uint32_t layout = 0, dim0 = 0, dim1 = 0, n_neurons = 0;
};

uint32_t image_side(const std::vector<uint32_t>& shape, uint32_t channels)
{
    uint32_t c = 1, h, w;
    if (shape.size() == 2) { h = shape[0]; w = shape[1]; }
    else if (shape.size() == 3) { c = shape[0]; h = shape[1]; w = shape[2]; }
    else throw pink_error("Not implemented yet.");
    if (h != w) throw pink_error("Images must be quadratic.");                              // generate_rotated_images.h:69-71
    if (c != channels) throw pink_error("image has " + std::to_string(c) + " channels, the SOM neurons have " + std::to_string(channels));
    return h;
}

// what Trainer and Mapper share: the configuration and the context, which is created with the first image
class Session
{
public:
    Session(SOM& som, uint32_t number_of_rotations, bool use_flip, Interpolation interpolation, bool use_gpu,
            uint32_t euclidean_distance_dim, EuclideanDistanceShape shape, DataType type)
     : m_som(som)
    {
        if (!use_gpu) throw pink_error("CPU execution is not supported by pink_b200 (there is no CPU fallback)");
        if (euclidean_distance_dim == 0) throw pink_error("euclidean_distance_dim not defined");   // DynamicTrainer.cpp:25
        if (number_of_rotations == 0 || (number_of_rotations != 1 && number_of_rotations % 4 != 0))
            throw pink_error("Number of rotations must be 1 or larger then 1 and divisible by 4");
        som.neuron_geometry(&m_cfg.channels, &m_cfg.neuron_dim);
        if (euclidean_distance_dim > m_cfg.neuron_dim) throw pink_error("Euclidean distance dimension larger than neuron dimension");
        m_cfg.n_neurons = som.n_neurons;
        m_cfg.ed_dim = euclidean_distance_dim;
        m_cfg.ed_shape = shape == EuclideanDistanceShape::QUADRATIC ? PINK_B200_QUADRATIC : PINK_B200_CIRCULAR;
        m_cfg.n_rotations = number_of_rotations;
        m_cfg.use_flip = use_flip;
        m_cfg.dist_type = type == DataType::FLOAT ? PINK_B200_FLOAT : (type == DataType::UINT16 ? PINK_B200_UINT16 : PINK_B200_UINT8);
        m_cfg.interpolation = interpolation == Interpolation::BILINEAR ? PINK_B200_BILINEAR : PINK_B200_NEAREST_NEIGHBOR;
        m_cfg.world_size = 1;
    }
    ~Session() { pink_b200_destroy(m_ctx); }
    Session(const Session&) = delete;
    Session& operator=(const Session&) = delete;

    // returns true when the context was created by this call
    bool open(const std::vector<uint32_t>& image_shape)
    {
        const uint32_t side = image_side(image_shape, m_cfg.channels);
        if (m_ctx) {
            if (side != m_cfg.image_dim) throw pink_error("all images must have the size of the first one");
            return false;
        }
        m_cfg.image_dim = side;
        check(pink_b200_create(&m_cfg, &m_ctx));
        check(pink_b200_set_som(m_ctx, m_som.data.data()));
        return true;
    }
    pink_b200_ctx* ctx() const { return m_ctx; }
    SOM& som() { return m_som; }
    size_t image_size() const { return (size_t)m_cfg.channels * m_cfg.image_dim * m_cfg.image_dim; }

private:
    SOM& m_som;
    pink_b200_config m_cfg{};
    pink_b200_ctx* m_ctx = nullptr;
};

class Trainer
{
public:
    Trainer(SOM& som, const py::object& distribution_function, int /*verbosity*/, uint32_t number_of_rotations, bool use_flip,
            float max_update_distance, Interpolation interpolation, bool use_gpu, uint32_t euclidean_distance_dim,
            EuclideanDistanceShape shape, DataType type)
     : m_session(som, number_of_rotations, use_flip, interpolation, use_gpu, euclidean_distance_dim, shape, type)
    {
        // factor(i, j) = f(distance(i, j)) if max_update_distance <= 0 or distance < max_update_distance, else 0
        // (TrainerCommon, src/SelfOrganizingMapLib/Trainer.h:69-76).  The callable is evaluated once per
        // DISTINCT map distance -- a SOM grid has few -- and the library looks the factor up by distance class:
        // the same factors as N^2 calls give, without an N x N table.
        const uint32_t classes = pink_b200_distance_classes(som.layout, som.dim0, som.dim1, 1, nullptr, 0);
        std::vector<float> distance(classes);
        pink_b200_distance_classes(som.layout, som.dim0, som.dim1, 1, distance.data(), classes);
        m_factors.resize(classes);
        const bool native = py::isinstance<GaussianFunctor>(distribution_function);
        const GaussianFunctor* g = native ? distribution_function.cast<const GaussianFunctor*>() : nullptr;
        for (uint32_t c = 0; c < classes; ++c) {
            const float d = distance[c];
            m_factors[c] = (max_update_distance <= 0 || d < max_update_distance)
                         ? (native ? (*g)(d) : distribution_function(d).cast<float>()) : 0.0f;
        }
    }

    // One image (src/pink/DynamicTrainer.h:110-120).  Nothing of a training step can be observed before
    // update_som() / get_update_info(), so the images are collected and handed to the device kDefer at a time:
    // whole batches of steps run in one launch instead of one launch sequence per image.
    void call(const Data& data)
    {
        prepare(data.shape);
        m_pending.insert(m_pending.end(), data.data.begin(), data.data.end());
        if (++m_n_pending == kDefer) flush();
    }

    // many images in one call: (n, id, id) or (n, C, id, id)
    void train(const py::array_t<float, py::array::c_style | py::array::forcecast>& images)
    {
        if (images.ndim() < 3) throw pink_error("images must have shape (n, id, id) or (n, C, id, id)");
        std::vector<uint32_t> shape(images.shape() + 1, images.shape() + images.ndim());
        prepare(shape);
        flush();
        check(pink_b200_train(m_session.ctx(), images.data(), (uint64_t)images.shape(0)));
    }

    // copies the trained weights into the SOM's storage (Trainer.h:306-309)
    void update_som()
    {
        if (!m_session.ctx()) return;
        flush();
        check(pink_b200_synchronize(m_session.ctx()));
        check(pink_b200_get_som(m_session.ctx(), m_session.som().data.data()));
    }

    py::array_t<uint32_t> get_update_info()
    {
        py::array_t<uint32_t> out((ssize_t)m_session.som().n_neurons);
        std::memset(out.mutable_data(), 0, out.size() * sizeof(uint32_t));
        if (m_session.ctx()) {
            flush();
            check(pink_b200_get_update_counts(m_session.ctx(), out.mutable_data()));
        }
        return out;
    }

private:
    static constexpr uint32_t kDefer = 16;          // images collected before they go to the device

    // the collected images, in order (pink_b200_train has taken them out of the buffer when it returns: pageable memory)
    void flush()
    {
        if (m_n_pending == 0) return;
        const uint32_t n = m_n_pending;
        m_n_pending = 0;
        const int rc = pink_b200_train(m_session.ctx(), m_pending.data(), n);
        m_pending.clear();
        check(rc);
    }

    void prepare(const std::vector<uint32_t>& image_shape)
    {
        if (m_session.open(image_shape)) {
            const SOM& som = m_session.som();
            check(pink_b200_set_update_lut(m_session.ctx(), som.layout, som.dim0, som.dim1, 1, m_factors.data(),
                                           (uint32_t)m_factors.size()));
        }
    }
    Session m_session;
    std::vector<float> m_factors;
    std::vector<float> m_pending;                   // images given to call() that have not gone to the device yet
    uint32_t m_n_pending = 0;
};

class Mapper
{
public:
    Mapper(SOM& som, int /*verbosity*/, uint32_t number_of_rotations, bool use_flip, Interpolation interpolation, bool use_gpu,
           uint32_t euclidean_distance_dim, EuclideanDistanceShape shape, DataType type)
     : m_session(som, number_of_rotations, use_flip, interpolation, use_gpu, euclidean_distance_dim, shape, type)
    {}

    // (distances, best transforms) as two lists, like the reference's tuple of vectors
    py::tuple call(const Data& data)
    {
        m_session.open(data.shape);
        const size_t N = m_session.som().n_neurons;
        std::vector<float> dist(N);
        std::vector<uint32_t> rot(N);
        check(pink_b200_map(m_session.ctx(), data.data.data(), 1, dist.data(), rot.data()));
        return py::make_tuple(py::cast(dist), py::cast(rot));
    }

    py::tuple map(const py::array_t<float, py::array::c_style | py::array::forcecast>& images)
    {
        if (images.ndim() < 3) throw pink_error("images must have shape (n, id, id) or (n, C, id, id)");
        std::vector<uint32_t> shape(images.shape() + 1, images.shape() + images.ndim());
        m_session.open(shape);
        const ssize_t n = images.shape(0), N = (ssize_t)m_session.som().n_neurons;
        py::array_t<float> dist({n, N});
        py::array_t<uint32_t> rot({n, N});
        check(pink_b200_map(m_session.ctx(), images.data(), (uint64_t)n, dist.mutable_data(), rot.mutable_data()));
        return py::make_tuple(dist, rot);
    }

private:
    Session m_session;
};

} // namespace

PYBIND11_MODULE(_pink, m)
{
    m.doc() = "Parallelized rotation and flipping INvariant Kohonen maps (PINK) -- B200 library";
    m.attr("__version__") = std::string("2.5 (") + pink_b200_version() + ")";
    py::register_exception<pink_error>(m, "PinkError", PyExc_RuntimeError);

    py::enum_<Interpolation>(m, "Interpolation")
        .value("NEAREST_NEIGHBOR", Interpolation::NEAREST_NEIGHBOR)
        .value("BILINEAR", Interpolation::BILINEAR)
        .export_values();
    py::enum_<DataType>(m, "DataType")
        .value("FLOAT", DataType::FLOAT)
        .value("UINT16", DataType::UINT16)
        .value("UINT8", DataType::UINT8)
        .export_values();
    py::enum_<Layout>(m, "Layout")
        .value("CARTESIAN", Layout::CARTESIAN)
        .value("HEXAGONAL", Layout::HEXAGONAL)
        .export_values();
    py::enum_<EuclideanDistanceShape>(m, "EuclideanDistanceShape")
        .value("QUADRATIC", EuclideanDistanceShape::QUADRATIC)
        .value("CIRCULAR", EuclideanDistanceShape::CIRCULAR)
        .export_values();

    py::class_<GaussianFunctor>(m, "GaussianFunctor")
        .def(py::init<float, float>(), py::arg("sigma") = 1.1, py::arg("damping") = 0.2)
        .def("__call__", [](const GaussianFunctor& f, float d) { return f(d); });

    py::class_<Data>(m, "Data", py::buffer_protocol())
        .def(py::init<const py::buffer&, const std::string&, const std::string&>(),
             py::arg().noconvert(), py::arg("data_type") = "float32", py::arg("layout") = "cartesian-2d")
        .def_buffer([](Data& d) { return float_buffer_info(d.data, d.shape); });

    py::class_<SOM>(m, "SOM", py::buffer_protocol())
        .def(py::init<const py::buffer&, const std::string&, const std::string&, const std::string&>(),
             py::arg().noconvert(), py::arg("data_type") = "float32", py::arg("som_layout") = "cartesian-2d",
             py::arg("neuron_layout") = "cartesian-2d")
        .def_buffer([](SOM& s) { return float_buffer_info(s.data, s.shape); })
        .def("get_som_layout", [](const SOM& s) { return s.som_layout; });

    py::class_<Trainer>(m, "Trainer")
        .def(py::init<SOM&, const py::object&, int, uint32_t, bool, float, Interpolation, bool, uint32_t,
                      EuclideanDistanceShape, DataType>(),
             py::arg("som"), py::arg("distribution_function") = GaussianFunctor(1.1f, 0.2f), py::arg("verbosity") = 0,
             py::arg("number_of_rotations") = 360UL, py::arg("use_flip") = true, py::arg("max_update_distance") = -1.0,
             py::arg("interpolation") = Interpolation::BILINEAR, py::arg("use_gpu") = true,
             py::arg("euclidean_distance_dim"), py::arg("euclidean_distance_shape") = EuclideanDistanceShape::QUADRATIC,
             py::arg("euclidean_distance_type") = DataType::UINT8, py::keep_alive<1, 2>())
        .def("__call__", &Trainer::call)
        .def("train", &Trainer::train)
        .def("update_som", &Trainer::update_som)
        .def("get_update_info", &Trainer::get_update_info);

    py::class_<Mapper>(m, "Mapper")
        .def(py::init<SOM&, int, uint32_t, bool, Interpolation, bool, uint32_t, EuclideanDistanceShape, DataType>(),
             py::arg("som"), py::arg("verbosity") = 0, py::arg("number_of_rotations") = 360UL, py::arg("use_flip") = true,
             py::arg("interpolation") = Interpolation::BILINEAR, py::arg("use_gpu") = true,
             py::arg("euclidean_distance_dim"), py::arg("euclidean_distance_shape") = EuclideanDistanceShape::QUADRATIC,
             py::arg("euclidean_distance_type") = DataType::UINT8, py::keep_alive<1, 2>())
        .def("__call__", &Mapper::call)
        .def("map", &Mapper::map);
}
