// The loop of aeon's examples/cpp_iterator/iterator.cpp on the B200 library: same calls, `aeon.hpp` replaced by
// `aeon_b200.hpp`.  aeon builds its configuration as a nlohmann::json object; that library is not part of this
// tree, so the configuration is given as JSON text, and through a small object with dump() to show that a JSON
// object is accepted as well.
//
// usage: iterator_example <directory with flowers.jpg and img_2112_70.jpg> <record count> [device_output]
// prints one line per batch: index, buffer count, first label, checksum of the first image.
#include <cstdint>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>

#include "aeon_b200.hpp"

using std::cout;
using std::endl;
using std::string;

using nervana::loader;
using nervana::loader_factory;

struct json_text // stands in for nlohmann::json: anything with dump()
{
    string text;
    string dump() const { return text; }
};

static string generate_manifest_file(const string& dir, size_t record_count)
{
    const string manifest_name = dir + "/manifest_cpp_iterator.txt";
    const char*  image_files[] = {"flowers.jpg", "img_2112_70.jpg"};
    std::ofstream f(manifest_name);
    f << "@FILE\tSTRING\n";
    for (size_t i = 0; i < record_count; i++)
        f << image_files[i % 2] << "\t" << std::to_string(i % 2) << "\n";
    return manifest_name;
}

int main(int argc, char** argv)
{
    if (argc < 3)
        return 2;
    const string manifest_root = argv[1];
    const size_t records       = std::stoul(argv[2]);
    const string manifest      = generate_manifest_file(manifest_root, records);
    const int    height = 32, width = 32;
    const size_t batch_size = 4;

    json_text config{"{\"manifest_root\": \"" + manifest_root + "\", \"manifest_filename\": \"" + manifest + "\", \"batch_size\": " +
                     std::to_string(batch_size) + ", \"iteration_mode\": \"ONCE\", \"etl\": [{\"type\": \"image\", \"height\": " +
                     std::to_string(height) + ", \"width\": " + std::to_string(width) +
                     ", \"channel_major\": false}, {\"type\": \"label\", \"binary\": false}], \"augmentation\": [{\"type\": \"image\", "
                     "\"flip_enable\": true}]}"};
    try
    {
        loader_factory          factory;
        std::shared_ptr<loader> train_set = factory.get_loader(config);

        cout << "batch size: " << train_set->batch_size() << endl;
        cout << "batch count: " << train_set->batch_count() << endl;
        cout << "record count: " << train_set->record_count() << endl;
        for (const auto& ns : train_set->get_names_and_shapes())
        {
            cout << "buffer " << ns.first << " " << ns.second.get_otype().get_name() << " [";
            for (size_t v : ns.second.get_shape())
                cout << " " << v;
            cout << " ] bytes " << ns.second.get_byte_size() << endl;
        }

        int batch_no = 0;
        for (const auto& batch : *train_set)
        {
            const nervana::buffer_fixed_size_elements* image = batch["image"];
            const nervana::buffer_fixed_size_elements* label = batch["label"];
            uint32_t first_label = 0;
            std::memcpy(&first_label, label->get_item(0), sizeof(first_label));
            unsigned long sum = 0;
            for (size_t i = 0; i < image->get_stride(); ++i)
                sum += (unsigned char)image->get_item(0)[i];
            cout << "\tbatch " << batch_no << " [number of elements: " << batch.size() << "] label " << first_label << " sum " << sum
                 << " items " << image->get_item_count() << endl;
            batch_no++;
        }
        cout << "batches: " << batch_no << " position " << train_set->position() << endl;
        // a second pass gives the same number of batches (begin() resets)
        int again = 0;
        for (auto it = train_set->begin(); it != train_set->end(); ++it)
            again++;
        cout << "again: " << again << endl;
        try
        {
            factory.get_loader(string("{\"batch_size\": 4}"));
            cout << "no error" << endl;
        }
        catch (const std::exception& e)
        {
            cout << "error: " << e.what() << endl;
        }
    }
    catch (const std::exception& e)
    {
        cout << "failed: " << e.what() << endl;
        return 1;
    }
    return 0;
}
