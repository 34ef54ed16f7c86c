// Binary file formats and data order of the PINK command line tool, for the host
// program that drives the GPU library.  Formats: FILE_FORMATS.md:53-85 of the
// reference; writers src/SelfOrganizingMapLib/FileIO.h:19-49 and
// src/Pink/main_generic.h:131-162,185-196; readers
// src/SelfOrganizingMapLib/DataIterator.h, DataIteratorShuffled.h:41-74,
// SOM.h:87-96, src/UtilitiesLib/get_file_header.cpp:11-31.
//
// All files are a sequence of native-endian 32-bit integers followed by raw
// float32 data, optionally preceded by text lines starting with '#'.
#pragma once

#include <algorithm>
#include <cstdint>
#include <fstream>
#include <numeric>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

namespace pinkhost {

// Text lines starting with '#' in front of the binary part; the line
// "# END OF HEADER" ends them even if more '#' lines follow.  Leaves the stream
// at the first byte after the header (or where it was if there is none).
inline std::string read_text_header(std::istream& is)
{
    std::string header, line;
    std::streampos keep = is.tellg();
    while (std::getline(is, line) && !line.empty() && line[0] == '#') {
        keep = is.tellg();
        header += line + '\n';
        if (line == "# END OF HEADER") break;
    }
    is.clear();
    is.seekg(keep, is.beg);
    return header;
}

inline int read_int(std::istream& is)
{
    int v = 0;
    is.read(reinterpret_cast<char*>(&v), sizeof(int));
    if (!is) throw std::runtime_error("unexpected end of file in the binary header");
    return v;
}

inline void write_int(std::ostream& os, int v) { os.write(reinterpret_cast<const char*>(&v), sizeof(int)); }

// <version> 0 <data type> <number of entries> <layout> <dimensionality> <dims...> <data>
struct DataFile
{
    std::string text_header;
    int version = 0, file_type = 0, data_type = 0, entries = 0, layout = 0;
    std::vector<int> dims;            // (height, width) or (channels, height, width)
    std::streamoff data_offset = 0;   // first byte of entry 0
    size_t entry_floats = 0;

    uint32_t channels() const { return dims.size() == 3 ? (uint32_t)dims[0] : 1u; }
    uint32_t side() const { return (uint32_t)dims.back(); }
};

inline DataFile open_data_file(std::istream& is)
{
    DataFile f;
    f.text_header = read_text_header(is);
    f.version = read_int(is);
    f.file_type = read_int(is);
    f.data_type = read_int(is);
    f.entries = read_int(is);
    f.layout = read_int(is);
    const int dimensionality = read_int(is);
    if (dimensionality < 1 || dimensionality > 3) throw std::runtime_error("data dimensionality must be 1, 2 or 3");
    f.entry_floats = 1;
    for (int i = 0; i < dimensionality; ++i) {
        f.dims.push_back(read_int(is));
        if (f.dims.back() <= 0) throw std::runtime_error("data dimensions must be positive");
        f.entry_floats *= (size_t)f.dims.back();
    }
    f.data_offset = is.tellg();
    // the reference's messages (src/UtilitiesLib/InputData.cpp:490-493)
    if (f.version != 2) throw std::runtime_error("Please use file format version 2 as data input.");
    if (f.file_type != 0) throw std::runtime_error("Please use file type 0 as data input.");
    if (f.data_type != 0) throw std::runtime_error("Only data_type = 0 (float, single precision) is supported.");
    if (f.entries <= 0) throw std::runtime_error("Number of data entries must be larger than 0.");
    return f;
}

inline void read_entry(std::istream& is, const DataFile& f, uint32_t index, float* dst)
{
    is.seekg(f.data_offset + (std::streamoff)((uint64_t)index * f.entry_floats * sizeof(float)), is.beg);
    is.read(reinterpret_cast<char*>(dst), (std::streamsize)(f.entry_floats * sizeof(float)));
    if (!is) throw std::runtime_error("unexpected end of the data file");
}

// Order in which one pass presents the entries: 0..n-1, or that list shuffled by
// std::shuffle with an mt19937 seeded from one draw of default_random_engine(seed)
// -- the reference's generator chain, so the same seed gives the same order with
// the same C++ standard library.  The training loop passes seed + pass index.
inline std::vector<uint32_t> entry_order(uint32_t n, uint64_t seed, bool shuffle)
{
    std::vector<uint32_t> order(n);
    std::iota(order.begin(), order.end(), 0u);
    if (shuffle) {
        std::default_random_engine engine(seed);
        std::mt19937 gen(engine());
        std::shuffle(order.begin(), order.end(), gen);
    }
    return order;
}

// <version> 1 <data type> <som layout> <som dimensionality> <som dims> <neuron layout>
// <neuron dimensionality> <neuron dims> <data>.  The layout index is written as 0 also for
// hexagonal maps, as the reference does.
inline void write_som_file(const std::string& path, const std::string& text_header, const std::vector<int>& som_dims,
                           const std::vector<int>& neuron_dims, const float* data, size_t count)
{
    std::ofstream os(path, std::ios::binary);
    if (!os) throw std::runtime_error("Error opening " + path);
    os << text_header;
    write_int(os, 2); write_int(os, 1); write_int(os, 0);
    write_int(os, 0); write_int(os, (int)som_dims.size());
    for (int d : som_dims) write_int(os, d);
    write_int(os, 0); write_int(os, (int)neuron_dims.size());
    for (int d : neuron_dims) write_int(os, d);
    os.write(reinterpret_cast<const char*>(data), (std::streamsize)(count * sizeof(float)));
    if (!os) throw std::runtime_error("Error writing " + path);
}

struct SomFile
{
    std::string text_header;
    std::vector<int> som_dims, neuron_dims;
    std::vector<float> data;
};

// Reads the dimensions from the file (the reference skips a fixed 9 + som dimensionality
// integers, which is the same position for 2-dimensional neurons).
inline SomFile read_som_file(const std::string& path)
{
    std::ifstream is(path, std::ios::binary);
    if (!is) throw std::runtime_error("Error opening " + path);
    SomFile f;
    f.text_header = read_text_header(is);
    const int version = read_int(is), type = read_int(is), dtype = read_int(is);
    if (version != 2 || type != 1 || dtype != 0) throw std::runtime_error(path + " is not a version 2 float SOM file");
    (void)read_int(is);
    const int sd = read_int(is);
    if (sd < 1 || sd > 3) throw std::runtime_error("SOM dimensionality must be 1, 2 or 3");
    for (int i = 0; i < sd; ++i) f.som_dims.push_back(read_int(is));
    (void)read_int(is);
    const int nd = read_int(is);
    if (nd < 1 || nd > 3) throw std::runtime_error("neuron dimensionality must be 1, 2 or 3");
    size_t neuron = 1;
    for (int i = 0; i < nd; ++i) { f.neuron_dims.push_back(read_int(is)); neuron *= (size_t)f.neuron_dims.back(); }
    const std::streampos here = is.tellg();
    is.seekg(0, is.end);
    const size_t bytes = (size_t)(is.tellg() - here);
    is.seekg(here, is.beg);
    if (neuron == 0 || bytes % (neuron * sizeof(float)) != 0) throw std::runtime_error(path + ": data size does not match the neuron size");
    f.data.resize(bytes / sizeof(float));
    is.read(reinterpret_cast<char*>(f.data.data()), (std::streamsize)bytes);
    return f;
}

// <version> 2 <data type> <number of entries> <som layout> <som dimensionality> <som dims> <data>
inline void write_mapping_header(std::ostream& os, int entries, const std::vector<int>& som_dims)
{
    write_int(os, 2); write_int(os, 2); write_int(os, 0); write_int(os, entries);
    write_int(os, 0); write_int(os, (int)som_dims.size());
    for (int d : som_dims) write_int(os, d);
}

// <version> 3 <number of entries> <som layout> <som dimensionality> <som dims> <data>;
// one record per neuron: 1 byte flipped + float32 angle in radians.
inline void write_rot_flip_header(std::ostream& os, int entries, const std::vector<int>& som_dims)
{
    write_int(os, 2); write_int(os, 3); write_int(os, entries);
    write_int(os, 0); write_int(os, (int)som_dims.size());
    for (int d : som_dims) write_int(os, d);
}

// Image indices (0-based, counted over all passes) after which the reference's loop stores an
// intermediate map: the positions where its progress bar reports
// (src/UtilitiesLib/ProgressBar.h:21-76, src/Pink/main_generic.h:87-107).
inline std::vector<uint64_t> report_points(uint64_t total, int max_prints)
{
    std::vector<uint64_t> points;
    if (total == 0 || max_prints < 1) return points;
    const uint64_t prints = std::min<uint64_t>(total, (uint64_t)max_prints);
    const uint64_t section = total / prints, rest = total % prints;
    for (uint64_t next = section + (rest ? 1 : 0); next < total; next += section) points.push_back(next);
    return points;
}

} // namespace pinkhost
