// A small program written against the reference's class API (pink::SOM, pink::Data,
// pink::Trainer<..., float, true>, pink::Mapper<..., float, true>): trains a 3 x 3 map (and a 2 x 2 x 2 map) on the
// images of a binary file and prints the trained map, the update counts and the mapping of
// the first image as text, which the test compares with the CPU oracle.
#include "pink_b200.hpp"

#include <cstdio>
#include <fstream>

using namespace pink;

int main(int argc, char** argv)
{
    if (argc < 3) return 2;
    try {
        typedef CartesianLayout<2> L2;
        std::ifstream is(argv[1], std::ios::binary);
        int head[8];
        is.read(reinterpret_cast<char*>(head), sizeof(head));          // 2 0 0 n 0 2 h w
        const uint32_t n = (uint32_t)head[3], id = (uint32_t)head[7], nd = 12, ed = 7, rot = 8;
        std::ifstream ss(argv[2], std::ios::binary);
        std::vector<float> init(9 * nd * nd);
        ss.read(reinterpret_cast<char*>(init.data()), (std::streamsize)(init.size() * sizeof(float)));

        SOM<L2, L2, float> som(L2{{3, 3}}, L2{{nd, nd}}, init);
        Trainer<L2, L2, float, true> trainer(som, GaussianFunctor(1.1f, 0.2f), 0, rot, true, -1.0f, Interpolation::BILINEAR,
            ed, EuclideanDistanceShape::QUADRATIC, 256, DataType::UINT8);
        std::vector<Data<L2, float>> images;
        for (uint32_t i = 0; i < n; ++i) {
            std::vector<float> px(id * id);
            is.read(reinterpret_cast<char*>(px.data()), (std::streamsize)(px.size() * sizeof(float)));
            images.emplace_back(L2{{id, id}}, std::move(px));
            trainer(images.back());
        }
        trainer.update_som();
        std::printf("som");
        for (size_t i = 0; i < som.size(); ++i) std::printf(" %08x", *reinterpret_cast<const uint32_t*>(som.get_data_pointer() + i));
        std::printf("\ncounts");
        for (auto c : trainer.get_update_info()) std::printf(" %u", c);

        Mapper<L2, L2, float, true> mapper(som, 0, rot, true, Interpolation::BILINEAR, ed, EuclideanDistanceShape::QUADRATIC, 256,
            DataType::UINT8);
        auto result = mapper(images[0]);
        std::printf("\ndist");
        for (float v : std::get<0>(result)) std::printf(" %08x", *reinterpret_cast<const uint32_t*>(&v));
        std::printf("\nrot");
        for (auto v : std::get<1>(result)) std::printf(" %u", v);
        std::printf("\n");

        // error behaviour: the reference's messages
        try {
            Trainer<L2, L2, float, true> bad(som, GaussianFunctor(1.1f, 0.2f), 0, 6, true, -1.0f, Interpolation::BILINEAR, ed);
            std::printf("error none\n");
        } catch (pink::exception const& e) {
            std::printf("error %s\n", e.what());
        }

        // a three-dimensional map (2 x 2 x 2 neurons) trained on the first two images
        typedef CartesianLayout<3> L3;
        std::vector<float> init3(init.begin(), init.begin() + 8 * nd * nd);
        SOM<L3, L2, float> som3(L3{{2, 2, 2}}, L2{{nd, nd}}, init3);
        Trainer<L3, L2, float, true> trainer3(som3, GaussianFunctor(1.1f, 0.2f), 0, rot, true, -1.0f, Interpolation::BILINEAR,
            ed, EuclideanDistanceShape::QUADRATIC, 256, DataType::UINT8);
        for (uint32_t i = 0; i < 2 && i < n; ++i) trainer3(images[i]);
        trainer3.update_som();
        std::printf("som3");
        for (size_t i = 0; i < som3.size(); ++i) std::printf(" %08x", *reinterpret_cast<const uint32_t*>(som3.get_data_pointer() + i));
        std::printf("\n");
        return 0;
    } catch (std::exception const& e) {
        std::fprintf(stderr, "exception: %s\n", e.what());
        return 1;
    }
}
