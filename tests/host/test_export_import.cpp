// Reads a network in the reference's on-disk forms (the per-cell headers of its CPP_Quantization export and
// `.syntxt` parameter files, here the hand-formatted fixture under tests/golden/export_fixture) through
// n2d2_b200/host/ExportImport.hpp.
//
//   test_export_import --parse <dir>                              prints what was read, one "key value..." line each
//   test_export_import --run <dir> <stimuli.bin> <batch> <out>    builds the DeepNet from the headers (editing the
//                                                                 graph on the way), runs it on cuda:0 and writes the
//                                                                 logits (int32) to <out>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>

#include "../../n2d2_b200/host/ExportImport.hpp"

using namespace N2D2;

template <class T> static void line(const std::string& key, const std::vector<T>& v)
{
    std::cout << key;
    for (const auto& x : v) std::cout << ' ' << (long long)x;
    std::cout << '\n';
}

static void dump(const ExportedCell& c)
{
    const std::string p = c.identifier + ".";
    std::cout << p << "activation " << c.activation << '\n';
    std::cout << p << "weightBits " << c.weightBits << '\n';
    std::cout << p << "outputUnsigned " << c.outputUnsigned << '\n';
    std::cout << p << "mode " << (int)c.scaling.getMode() << '\n';
    std::cout << p << "fracBits " << c.scaling.getFractionalBits() << '\n';
    std::cout << p << "isClipped " << (c.scaling.getIsClipped() ? 1 : 0) << '\n';
    for (const auto& kv : c.constants) std::cout << p << "const." << kv.first << ' ' << kv.second << '\n';
    for (const auto& kv : c.names) std::cout << p << "name." << kv.first << ' ' << kv.second << '\n';
    line(p + "biases", c.biases);
    line(p + "exportedBiases", c.exportedBiases);
    line(p + "weights", c.weights);
    n2d2b_scaling d;
    c.scaling.describe(d, (int)c.constant("NB_OUTPUTS"));
    const int n = (int)c.constant("NB_OUTPUTS");
    if (d.mult) line(p + "mult", std::vector<long long>(d.mult, d.mult + n));
    if (d.shift0) line(p + "shift0", std::vector<long long>(d.shift0, d.shift0 + n));
    if (d.shift1) line(p + "shift1", std::vector<long long>(d.shift1, d.shift1 + n));
    if (d.clip) line(p + "clip", std::vector<long long>(d.clip, d.clip + n));
}

int main(int argc, char** argv)
{
    if (argc < 3) { fprintf(stderr, "usage: see the top of the source file\n"); return 2; }
    const std::string dir = argv[2];
    try {
        const ExportedCell conv1 = loadExportedCell(dir + "/conv1.hpp"), pool1 = loadExportedCell(dir + "/pool1.hpp"),
                           conv2 = loadExportedCell(dir + "/conv2.hpp"), conv3 = loadExportedCell(dir + "/conv3_w4.hpp"),
                           sum1 = loadExportedCell(dir + "/sum1.hpp"), fc1 = loadExportedCell(dir + "/fc1.hpp");
        const auto synW = synTxtAsIntegers<std::int8_t>(loadSynTxt(dir + "/conv1_weights.syntxt"), -128, 127, "conv1 weights");
        const auto synB = synTxtAsIntegers<std::int32_t>(loadSynTxt(dir + "/conv1_biases.syntxt"), INT32_MIN, INT32_MAX, "conv1 biases");
        if (!strcmp(argv[1], "--parse")) {
            for (const ExportedCell* c : {&conv1, &pool1, &conv2, &conv3, &sum1, &fc1}) dump(*c);
            line("syntxt.conv1.weights", synW);
            line("syntxt.conv1.biases", synB);
            // malformed input is an exception with the cell's name, like the reference's loaders
            bool threw = false;
            try { parseExportedCell("#define X_NB_OUTPUTS 2\nstatic const int32_t x_biases[X_NB_OUTPUTS] = {1, 2, 3};\n"); }
            catch (const std::runtime_error& e) { threw = std::string(e.what()).find("3 biases for 2 outputs") != std::string::npos; }
            std::cout << "malformed.threw " << (threw ? 1 : 0) << '\n';
            // weights below four bits as the QAT export packs them (first value in the high bits, every run of channels
            // padded to whole bytes; one-bit weights store -1 as 0)
            const ExportedCell w2 = parseExportedCell(
                "#define Q2_NB_OUTPUTS 1\n#define Q2_NB_CHANNELS 5\n#define Q2_KERNEL_WIDTH 1\n#define Q2_KERNEL_HEIGHT 1\n"
                "static const data<2> q2_weights[Q2_WEIGHTS_SIZE] N2D2_SECTION_ATTRIBUTE(N2D2_SECTION_NN_WEIGHTS) = {0x72, 0x40, \n};\n");
            line("w2.weights", w2.weights);
            const ExportedCell w1 = parseExportedCell(
                "#define Q1_NB_OUTPUTS 1\n#define Q1_NB_CHANNELS 9\n#define Q1_KERNEL_WIDTH 1\n#define Q1_KERNEL_HEIGHT 1\n"
                "static const data<1> q1_weights[Q1_WEIGHTS_SIZE] N2D2_SECTION_ATTRIBUTE(N2D2_SECTION_NN_WEIGHTS) = {0x9b, 0x80, \n};\n");
            line("w1.weights", w1.weights);
            return 0;
        }
        if (strcmp(argv[1], "--run") || argc < 6) { fprintf(stderr, "usage: see the top of the source file\n"); return 2; }
        const unsigned batch = (unsigned)atoi(argv[4]);
        std::ifstream sf(argv[3], std::ios::binary);
        std::vector<std::uint8_t> stimuli((size_t)batch * 12 * 12);
        sf.read((char*)stimuli.data(), (std::streamsize)stimuli.size());
        if (!sf) { fprintf(stderr, "short stimuli file\n"); return 2; }

        DeepNet deepNet(1, 12, 12);
        auto c1 = convCellFromExport(conv1);
        auto p1 = poolCellFromExport(pool1);
        auto c2 = convCellFromExport(conv2);
        auto c3 = convCellFromExport(conv3);
        auto s1 = elemWiseCellFromExport(sum1);
        auto f1 = fcCellFromExport(fc1);
        // conv1's parameters once more from the .syntxt files: same network
        if (c1->getWeights() != synW || c1->getBiases() != synB) { fprintf(stderr, ".syntxt and header disagree\n"); return 1; }
        // wiring as the export's network description gives it; conv2 first goes straight after conv1 and the pooling
        // cell is put between them afterwards, then a stray cell is added and removed again (graph editing as the
        // post-training quantization does it)
        deepNet.addCell(c1, {});
        deepNet.addCell(c2, {c1});
        deepNet.addCellBetween(p1, c1, c2);
        deepNet.addCell(c3, {c2});
        deepNet.addCell(s1, {c3, c2});
        deepNet.addCell(f1, {s1});
        auto stray = std::make_shared<ScalingCell>("stray", 16, Scaling::singleShiftScaling(std::vector<unsigned char>(16, 2), false, {}));
        deepNet.addCellAfter(stray, c2);
        if (deepNet.getParentCells("conv3_w4")[0]->getName() != "stray" || deepNet.getChildCells("stray").size() != 2) {
            fprintf(stderr, "addCellAfter did not re-wire the children\n");
            return 1;
        }
        deepNet.removeCell(stray);
        const auto parents = deepNet.getParentCells("sum1");
        if (parents.size() != 2 || parents[0]->getName() != "conv3_w4" || parents[1]->getName() != "conv2"
            || deepNet.getParentCells("conv2")[0]->getName() != "pool1" || c2->getNbChannels() != 8 || c2->getOutputsWidth() != 4) {
            fprintf(stderr, "graph editing left the wrong wiring\n");
            return 1;
        }
        deepNet.initialize(batch);
        const std::vector<int> logits = deepNet.test(stimuli, batch);
        std::ofstream of(argv[5], std::ios::binary);
        of.write((const char*)logits.data(), (std::streamsize)(logits.size() * sizeof(int)));
        printf("ran %u stimuli through %zu layers\n", batch, deepNet.getLayers().size() - 1);
        return 0;
    } catch (const std::exception& e) {
        fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
