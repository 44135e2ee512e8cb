// Readers for the two on-disk forms in which the reference hands over a quantized network:
//
//   * the per-cell headers its CPP / CPP_Quantization export writes (`<cell>.hpp`): geometry as
//     `#define <CELL>_<KEY> value` (src/Export/CPP/CPP_ConvCellExport.cpp:75-135), `<cell>_biases[]`
//     (:145-174, with the single-shift rounding half pre-added as "b + h",
//     src/Export/CellExport.cpp:100-117), `<cell>_weights[]` in [output][ky][kx][channel] order
//     (:251-260; sub-byte weights of QAT nets as `data<N>` hex bytes, first value in the high bits, every
//     (output, ky, kx) run of channels padded to a whole byte, :419-607), the activation type
//     (src/Export/CPP/CPP_CellExport.cpp:53-83) and the `<CELL>_SCALING` object (:110-241);
//   * the `.syntxt` parameter files of Cell::exportFreeParameters (src/Cell/ConvCell.cpp:299-411): one
//     line per output, channel by channel, kernel values x-fastest; biases one per line.
//
// Nothing here runs the reference or needs its sources: the formats are plain text.  The result feeds
// the host classes of N2D2.hpp (Scaling, ConvCell::setWeights ...), i.e. the C ABI.
#pragma once

#include <cctype>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <fstream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "N2D2.hpp"

namespace N2D2 {

struct ExportedCell {
    std::string identifier;                        // C identifier of the cell ("conv1_1x1")
    std::map<std::string, long long> constants;    // NB_OUTPUTS, KERNEL_WIDTH, STRIDE_X, ... (cell prefix removed)
    std::map<std::string, std::string> names;      // defines whose value is an identifier: POOLING (Max | Average), ELEM_OP ...
    std::string activation = "Linear";             // Linear | Rectifier | Saturation
    Scaling scaling;                               // NONE when the header declares NoScaling
    int outputUnsigned = -1;                       // 1 / 0 when the scaling type states it, else -1
    bool hasBiases = false, hasWeights = false;
    std::vector<std::int64_t> exportedBiases;      // as written (rounding half of a single shift included)
    std::vector<std::int32_t> biases;              // the cell's own biases (that half removed again)
    int weightBits = 8;                            // storage width of the weights in the header
    std::vector<std::int8_t> weights;              // [output][ky][kx][channel], one value per element

    long long constant(const std::string& key) const
    {
        auto it = constants.find(key);
        if (it == constants.end()) throw std::runtime_error("exported cell " + identifier + ": no constant " + key);
        return it->second;
    }
    bool has(const std::string& key) const { return constants.count(key) != 0; }
};

namespace export_detail {

inline std::string trim(const std::string& s)
{
    std::size_t a = 0, b = s.size();
    while (a < b && std::isspace((unsigned char)s[a])) ++a;
    while (b > a && std::isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
}

inline std::string upper(std::string s)
{
    for (char& c : s) c = (char)std::toupper((unsigned char)c);
    return s;
}

// "12", "-3", "0x1f", "12 + 64", "3f" (float suffix) -> value; integers only unless `real` is given
inline bool parseNumber(const std::string& tok, long long* integer, double* real)
{
    const std::string t = trim(tok);
    if (t.empty()) return false;
    // a sum of terms (the exported single-shift bias: "b + half")
    std::size_t plus = t.find('+', 1);
    if (plus != std::string::npos && t.find_first_of("eE") == std::string::npos) {
        long long a = 0, b = 0;
        double ra = 0, rb = 0;
        if (!parseNumber(t.substr(0, plus), &a, &ra) || !parseNumber(t.substr(plus + 1), &b, &rb)) return false;
        if (integer) *integer = a + b;
        if (real) *real = ra + rb;
        return true;
    }
    char* end = nullptr;
    if (t.size() > 2 && t[0] == '0' && (t[1] == 'x' || t[1] == 'X')) {
        const long long v = std::strtoll(t.c_str(), &end, 16);
        if (*end) return false;
        if (integer) *integer = v;
        if (real) *real = (double)v;
        return true;
    }
    const long long v = std::strtoll(t.c_str(), &end, 10);
    if (*end == 0 || (*end && std::string(end).find_first_not_of("uUlL") == std::string::npos)) {
        if (integer) *integer = v;
        if (real) *real = (double)v;
        return true;
    }
    const double d = std::strtod(t.c_str(), &end);
    if (*end && std::string(end) != "f" && std::string(end) != "F") return false;
    if (integer) {
        if (std::fabs(d - std::round(d)) > 0.01) return false;   // CellExport::getIntFreeParameter's tolerance
        *integer = (long long)std::llround(d);
    }
    if (real) *real = d;
    return true;
}

// Splits "a, b, {c, d}, e" at top-level commas (nested braces and template brackets stay together).
inline std::vector<std::string> splitTopLevel(const std::string& s)
{
    std::vector<std::string> out;
    int depth = 0;
    std::string cur;
    for (char c : s) {
        if (c == '{' || c == '<' || c == '(') ++depth;
        if (c == '}' || c == '>' || c == ')') --depth;
        if (c == ',' && depth == 0) {
            if (!trim(cur).empty()) out.push_back(trim(cur));
            cur.clear();
        } else {
            cur += c;
        }
    }
    if (!trim(cur).empty()) out.push_back(trim(cur));
    return out;
}

// Text between the '{' that follows `from` and its matching '}' (empty when the statement ends first).
inline bool bracedAfter(const std::string& text, std::size_t from, std::string* inner, std::size_t* endPos)
{
    const std::size_t semi = text.find(';', from);
    const std::size_t open = text.find('{', from);
    if (open == std::string::npos || (semi != std::string::npos && semi < open)) return false;
    int depth = 0;
    for (std::size_t i = open; i < text.size(); ++i) {
        if (text[i] == '{') ++depth;
        if (text[i] == '}' && --depth == 0) {
            *inner = text.substr(open + 1, i - open - 1);
            if (endPos) *endPos = i + 1;
            return true;
        }
    }
    throw std::runtime_error("exported header: unbalanced braces");
}

inline std::vector<long long> integerList(const std::string& inner, const char* what)
{
    std::vector<long long> v;
    for (const std::string& tok : splitTopLevel(inner)) {
        long long x = 0;
        if (!parseNumber(tok, &x, nullptr)) throw std::runtime_error(std::string("exported header: bad value '") + tok + "' in " + what);
        v.push_back(x);
    }
    return v;
}

inline std::vector<Float_T> realList(const std::string& inner, const char* what)
{
    std::vector<Float_T> v;
    for (const std::string& tok : splitTopLevel(inner)) {
        double x = 0;
        if (!parseNumber(tok, nullptr, &x)) throw std::runtime_error(std::string("exported header: bad value '") + tok + "' in " + what);
        v.push_back((Float_T)x);
    }
    return v;
}

}  // namespace export_detail

// Parses the text of one exported `<cell>.hpp`.
inline ExportedCell parseExportedCell(const std::string& text)
{
    using namespace export_detail;
    ExportedCell cell;
    // ---- arrays give the identifier: "<id>_biases[" / "<id>_weights["
    auto arrayAt = [&](const std::string& suffix, std::string* id, std::string* type, std::string* inner) -> bool {
        const std::size_t pos = text.find(suffix + "[");
        if (pos == std::string::npos) return false;
        std::size_t b = pos;
        while (b > 0 && (std::isalnum((unsigned char)text[b - 1]) || text[b - 1] == '_')) --b;
        *id = text.substr(b, pos - b);
        // the element type: what stands between "static const" and the identifier
        const std::size_t sc = text.rfind("const", b);
        *type = sc == std::string::npos ? "" : trim(text.substr(sc + 5, b - sc - 5));
        const std::size_t eq = text.find('=', pos);
        if (eq == std::string::npos || !bracedAfter(text, eq, inner, nullptr))
            throw std::runtime_error("exported header: array " + *id + suffix + " has no initialiser");
        return true;
    };
    std::string idB, idW, typeB, typeW, innerB, innerW;
    cell.hasBiases = arrayAt("_biases", &idB, &typeB, &innerB);
    cell.hasWeights = arrayAt("_weights", &idW, &typeW, &innerW);
    if (cell.hasBiases && cell.hasWeights && idB != idW)
        throw std::runtime_error("exported header: biases belong to " + idB + ", weights to " + idW);
    cell.identifier = cell.hasWeights ? idW : idB;

    // ---- #define <PREFIX>_<KEY> value
    std::string prefix = upper(cell.identifier);
    std::istringstream lines(text);
    std::string line;
    while (std::getline(lines, line)) {
        const std::string t = trim(line);
        if (t.compare(0, 7, "#define") != 0) continue;
        std::istringstream ls(t.substr(7));
        std::string name, value;
        ls >> name;
        std::getline(ls, value);
        value = trim(value);
        if (prefix.empty()) {
            // a cell without parameters (pooling, element-wise): the prefix is what precedes _NB_OUTPUTS
            const std::size_t p = name.find("_NB_OUTPUTS");
            if (p != std::string::npos && p + 11 == name.size()) {
                prefix = name.substr(0, p);
                // only the upper-case form survives in such a header; the lower-case one is the usual cell name
                cell.identifier = prefix;
                for (char& ch : cell.identifier) ch = (char)std::tolower((unsigned char)ch);
            }
        }
        if (prefix.empty() || name.compare(0, prefix.size() + 1, prefix + "_") != 0) continue;
        const std::string key = name.substr(prefix.size() + 1);
        if (key == "ACTIVATION") {
            cell.activation = value;
            continue;
        }
        long long v = 0;
        if (parseNumber(value, &v, nullptr)) cell.constants[key] = v;
        else if (!value.empty() && value.find_first_of("(*") == std::string::npos) cell.names[key] = value;   // derived macros ("(A*B)") are skipped
    }
    if (prefix.empty()) throw std::runtime_error("exported header: no cell found (no arrays, no <CELL>_NB_OUTPUTS)");
    const std::size_t nbOutputs = (std::size_t)cell.constant("NB_OUTPUTS");

    // ---- <PREFIX>_SCALING
    {
        const std::string tag = " " + prefix + "_SCALING";
        std::size_t pos = text.find(tag);
        // the C-style legacy macros of the same header (<PREFIX>_SCALING_...) are not the object
        while (pos != std::string::npos && (std::isalnum((unsigned char)text[pos + tag.size()]) || text[pos + tag.size()] == '_'))
            pos = text.find(tag, pos + 1);
        if (pos != std::string::npos) {
            const std::size_t ns = text.rfind("N2D2_Export::", pos);
            if (ns == std::string::npos) throw std::runtime_error("exported header: " + prefix + "_SCALING without a type");
            const std::string type = trim(text.substr(ns + 13, pos - ns - 13));
            std::string kind = type, targs;
            const std::size_t lt = type.find('<');
            if (lt != std::string::npos) {
                kind = trim(type.substr(0, lt));
                targs = type.substr(lt + 1, type.rfind('>') - lt - 1);
            }
            std::vector<long long> ta;
            if (!targs.empty()) ta = integerList(targs, "scaling template arguments");
            std::string init;
            const bool hasInit = bracedAfter(text, pos, &init, nullptr);
            auto need = [&](bool ok) {
                if (!ok) throw std::runtime_error("exported header: malformed " + type + " " + prefix + "_SCALING");
            };
            auto spread = [&](auto v) { return std::vector<decltype(v)>(nbOutputs, v); };
            if (kind == "NoScaling") {
                cell.scaling = Scaling();
            } else if (kind == "FloatingPointScaling") {
                need(hasInit);
                const auto f = realList(init, "scaling");
                need(f.size() == 1);
                cell.scaling = Scaling::floatingPointScaling(spread(f[0]), false, {});
            } else if (kind == "FloatingPointClippingAndScaling") {
                need(hasInit);
                const auto f = realList(init, "scaling");
                need(f.size() == 2);
                cell.scaling = Scaling::floatingPointScaling(spread(f[0]), true, spread(f[1]));
            } else if (kind == "FloatingPointScalingPerChannel") {
                need(hasInit);
                auto f = realList(init, "scaling");
                need(f.size() == nbOutputs);
                cell.scaling = Scaling::floatingPointScaling(f, false, {});
            } else if (kind == "FloatingPointClippingAndScalingPerChannel" || kind == "FixedPointClippingAndScalingPerChannel") {
                need(hasInit);
                const auto parts = splitTopLevel(init);
                need(parts.size() == 2 && parts[0].front() == '{' && parts[1].front() == '{');
                const std::string a = parts[0].substr(1, parts[0].size() - 2), b = parts[1].substr(1, parts[1].size() - 2);
                auto clip = realList(b, "clipping");
                need(clip.size() == nbOutputs);
                if (kind[1] == 'l') {   // FloatingPoint...
                    auto f = realList(a, "scaling");
                    need(f.size() == nbOutputs);
                    cell.scaling = Scaling::floatingPointScaling(f, true, clip);
                } else {
                    need(ta.size() == 2);
                    const auto m = integerList(a, "scaling");
                    need(m.size() == nbOutputs);
                    cell.scaling = Scaling::fixedPointScaling(ScalingMode::FIXED_MULT32, (std::size_t)ta[1],
                                                              std::vector<std::int32_t>(m.begin(), m.end()), true, clip);
                }
            } else if (kind == "FixedPointScaling") {
                need(ta.size() == 2);
                cell.scaling = Scaling::fixedPointScaling(ScalingMode::FIXED_MULT32, (std::size_t)ta[1], spread((std::int32_t)ta[0]),
                                                          false, {});
            } else if (kind == "FixedPointScalingPerChannel") {
                need(hasInit && ta.size() == 2);
                const auto m = integerList(init, "scaling");
                need(m.size() == nbOutputs);
                cell.scaling = Scaling::fixedPointScaling(ScalingMode::FIXED_MULT32, (std::size_t)ta[1],
                                                          std::vector<std::int32_t>(m.begin(), m.end()), false, {});
            } else if (kind == "SingleShiftScaling") {
                need(ta.size() == 1);
                cell.scaling = Scaling::singleShiftScaling(spread((unsigned char)ta[0]), false, {});
            } else if (kind == "SingleShiftScalingPerChannel") {
                need(hasInit);
                const auto s = integerList(init, "scaling");
                need(s.size() == nbOutputs);
                cell.scaling = Scaling::singleShiftScaling(std::vector<unsigned char>(s.begin(), s.end()), false, {});
            } else if (kind == "DoubleShiftScaling") {
                need(ta.size() == 2);
                cell.scaling = Scaling::doubleShiftScaling(spread(std::make_pair((unsigned char)ta[0], (unsigned char)ta[1])), false, {});
            } else if (kind == "DoubleShiftScalingPerChannel") {
                need(hasInit && ta.size() == 2);
                cell.outputUnsigned = ta[1] ? 1 : 0;
                std::vector<std::pair<unsigned char, unsigned char> > pairs;
                for (const std::string& item : splitTopLevel(init)) {
                    // std::array<SUM_T, 3>{a, b, 2^(b-1)}
                    std::string in;
                    need(bracedAfter(item, 0, &in, nullptr));
                    const auto abh = integerList(in, "scaling");
                    need(abh.size() == 3);
                    pairs.emplace_back((unsigned char)abh[0], (unsigned char)abh[1]);
                }
                need(pairs.size() == nbOutputs);
                cell.scaling = Scaling::doubleShiftScaling(pairs, false, {});
            } else {
                throw std::runtime_error("exported header: unknown scaling type " + type);
            }
        }
    }

    // ---- biases: the export adds 2^(s-1) to the bias of a single-shift cell so that its run time only shifts
    if (cell.hasBiases) {
        const auto b = integerList(innerB, "biases");
        if (b.size() != nbOutputs) throw std::runtime_error("exported cell " + cell.identifier + ": " + std::to_string(b.size()) + " biases for " + std::to_string(nbOutputs) + " outputs");
        cell.exportedBiases.assign(b.begin(), b.end());
        n2d2b_scaling d;
        cell.scaling.describe(d, (int)nbOutputs);
        for (std::size_t o = 0; o < nbOutputs; ++o) {
            long long v = b[o];
            if (cell.scaling.getMode() == ScalingMode::SINGLE_SHIFT && d.shift0[o] > 0) v -= 1ll << (d.shift0[o] - 1);
            cell.biases.push_back((std::int32_t)v);
        }
    }

    // ---- weights
    if (cell.hasWeights) {
        const std::vector<long long> raw = integerList(innerW, "weights");
        int bits = 8;
        const std::size_t dpos = typeW.find("data<");
        if (dpos != std::string::npos) bits = std::atoi(typeW.c_str() + dpos + 5);
        if (bits != 8 && bits != 4 && bits != 2 && bits != 1)
            throw std::runtime_error("exported cell " + cell.identifier + ": unsupported weight storage of " + std::to_string(bits) + " bits");
        cell.weightBits = bits;
        if (bits == 8) {
            for (long long v : raw) {
                if (v < -128 || v > 255) throw std::runtime_error("exported cell " + cell.identifier + ": weight out of the 8-bit range");
                cell.weights.push_back((std::int8_t)v);
            }
        } else {
            // packed: every run of `run` values (the channels of one (output, ky, kx); for a fully-connected cell
            // the whole input) fills whole bytes, first value in the high bits, the tail padded with zeros
            if (cell.has("NB_GROUPS") && cell.constant("NB_GROUPS") > 1)
                throw std::runtime_error("exported cell " + cell.identifier + ": packed depthwise weights are not supported");
            const std::size_t channels = (std::size_t)cell.constant("NB_CHANNELS");
            const std::size_t taps = cell.has("KERNEL_WIDTH") ? (std::size_t)(cell.constant("KERNEL_WIDTH") * cell.constant("KERNEL_HEIGHT")) : 1;
            std::size_t run = channels;
            if (!cell.has("KERNEL_WIDTH") && cell.has("CHANNELS_HEIGHT"))
                run = channels * (std::size_t)(cell.constant("CHANNELS_HEIGHT") * cell.constant("CHANNELS_WIDTH"));
            const std::size_t perByte = 8 / bits, bytesPerRun = (run + perByte - 1) / perByte;
            if (raw.size() != nbOutputs * taps * bytesPerRun)
                throw std::runtime_error("exported cell " + cell.identifier + ": " + std::to_string(raw.size()) + " weight bytes, expected " + std::to_string(nbOutputs * taps * bytesPerRun));
            const int mask = (1 << bits) - 1, sign = 1 << (bits - 1);
            for (std::size_t r = 0; r < nbOutputs * taps; ++r)
                for (std::size_t i = 0; i < run; ++i) {
                    const int byte = (int)raw[r * bytesPerRun + i / perByte] & 0xff;
                    int v = (byte >> (bits * (perByte - 1 - i % perByte))) & mask;
                    if (bits == 1) v = v ? 1 : -1;           // the export stores -1 as 0
                    else if (v & sign) v -= 1 << bits;
                    cell.weights.push_back((std::int8_t)v);
                }
        }
    }
    return cell;
}

inline ExportedCell loadExportedCell(const std::string& path)
{
    std::ifstream f(path.c_str());
    if (!f.good()) throw std::runtime_error("Could not open exported cell header: " + path);
    std::stringstream ss;
    ss << f.rdbuf();
    return parseExportedCell(ss.str());
}

// A `.syntxt` parameter file: whitespace-separated numbers, returned in file order (conv / fc weights:
// [output][channel][ky][kx], i.e. what ConvCell::setWeights takes; biases: one per output).  A quantized
// network holds integral values in it; `integral` = false returns them unrounded for a float network.
inline std::vector<double> loadSynTxt(const std::string& path)
{
    std::ifstream f(path.c_str());
    if (!f.good()) throw std::runtime_error("Could not open synaptic file: " + path);
    std::vector<double> v;
    double x;
    while (f >> x) v.push_back(x);
    if (!f.eof()) throw std::runtime_error("Synaptic file " + path + " holds something that is not a number");
    return v;
}

template <class T> inline std::vector<T> synTxtAsIntegers(const std::vector<double>& v, long long lo, long long hi, const std::string& what)
{
    std::vector<T> out;
    out.reserve(v.size());
    for (double x : v) {
        if (std::fabs(x - std::round(x)) > 0.01)
            throw std::runtime_error(what + ": a non-integral parameter; the network must be quantized beforehand");
        const long long r = std::llround(x);
        if (r < lo || r > hi) throw std::runtime_error(what + ": parameter out of range");
        out.push_back((T)r);
    }
    return out;
}

// The exported weight order [output][ky][kx][channel] as the [output][channel][ky][kx] order of
// ConvCell::setWeights / FcCell::setWeights.
inline std::vector<std::int8_t> exportedWeightsAsOIHW(const ExportedCell& c, std::size_t channelsPerGroup, std::size_t kh, std::size_t kw)
{
    const std::size_t O = (std::size_t)c.constant("NB_OUTPUTS");
    if (c.weights.size() != O * kh * kw * channelsPerGroup)
        throw std::runtime_error("exported cell " + c.identifier + ": " + std::to_string(c.weights.size()) + " weights, expected " + std::to_string(O * kh * kw * channelsPerGroup));
    std::vector<std::int8_t> w(c.weights.size());
    for (std::size_t o = 0; o < O; ++o)
        for (std::size_t y = 0; y < kh; ++y)
            for (std::size_t x = 0; x < kw; ++x)
                for (std::size_t ch = 0; ch < channelsPerGroup; ++ch)
                    w[((o * channelsPerGroup + ch) * kh + y) * kw + x] = c.weights[((o * kh + y) * kw + x) * channelsPerGroup + ch];
    return w;
}

inline std::shared_ptr<Activation> exportedActivation(const ExportedCell& c, int saturationThreshold = 0)
{
    std::shared_ptr<Activation> a;
    if (c.activation == "Rectifier") a = std::make_shared<RectifierActivation>();
    else if (c.activation == "Saturation") a = std::make_shared<SaturationActivation>(saturationThreshold);
    else if (c.activation == "Linear") a = std::make_shared<LinearActivation>();
    else throw std::runtime_error("exported cell " + c.identifier + ": activation " + c.activation + " is not on the quantized path");
    a->setActivationScaling(c.scaling);
    return a;
}

// A ConvCell from an exported conv header (geometry, weights, biases, activation and scaling).
inline std::shared_ptr<ConvCell> convCellFromExport(const ExportedCell& c)
{
    const unsigned kw = (unsigned)c.constant("KERNEL_WIDTH"), kh = (unsigned)c.constant("KERNEL_HEIGHT");
    if ((c.has("SUB_SAMPLE_X") && c.constant("SUB_SAMPLE_X") != 1) || (c.has("SUB_SAMPLE_Y") && c.constant("SUB_SAMPLE_Y") != 1))
        throw std::domain_error("exported cell " + c.identifier + ": sub-sampling is not supported");
    const unsigned groups = c.has("NB_GROUPS") ? (unsigned)c.constant("NB_GROUPS") : 1;
    const int px = (int)c.constant("PADDING_X"), py = (int)c.constant("PADDING_Y");
    // the header gives the left / top padding; right / bottom follow from the output size it states
    const long long sx = c.constant("STRIDE_X"), sy = c.constant("STRIDE_Y"), dx = c.constant("DILATION_X"), dy = c.constant("DILATION_Y");
    const long long ox = c.constant("OUTPUTS_WIDTH"), oy = c.constant("OUTPUTS_HEIGHT");
    const long long needW = (ox - 1) * sx + dx * (kw - 1) + 1, needH = (oy - 1) * sy + dy * (kh - 1) + 1;
    int pr = (int)(needW - c.constant("CHANNELS_WIDTH") - px), pb = (int)(needH - c.constant("CHANNELS_HEIGHT") - py);
    if (pr < 0) pr = 0;
    if (pb < 0) pb = 0;
    auto cell = std::make_shared<ConvCell>(c.identifier, std::vector<unsigned>{kw, kh}, (unsigned)c.constant("NB_OUTPUTS"),
                                           std::vector<unsigned>{1, 1}, std::vector<unsigned>{(unsigned)sx, (unsigned)sy},
                                           std::vector<int>{px, py, pr, pb}, std::vector<unsigned>{(unsigned)dx, (unsigned)dy},
                                           exportedActivation(c));
    cell->setNbGroups(groups);
    cell->setWeights(exportedWeightsAsOIHW(c, (std::size_t)c.constant("NB_CHANNELS") / groups, kh, kw));
    if (!(c.has("NO_BIAS") && c.constant("NO_BIAS")) && c.hasBiases) cell->setBiases(c.biases);
    else if (c.hasBiases && c.scaling.getMode() == ScalingMode::SINGLE_SHIFT) cell->setBiases(c.biases);   // all zero once the half is removed
    cell->setQuantized(8);
    if (c.outputUnsigned >= 0) cell->setOutputUnsigned(c.outputUnsigned != 0);
    return cell;
}

// An FcCell from an exported fc header: the exported weights run over the input in (y, x, channel) order
// (src/Export/CPP/CPP_FcCellExport.cpp:143-161), FcCell::setWeights takes the reference's (channel, y, x).
inline std::shared_ptr<FcCell> fcCellFromExport(const ExportedCell& c)
{
    const std::size_t O = (std::size_t)c.constant("NB_OUTPUTS"), C = (std::size_t)c.constant("NB_CHANNELS");
    const std::size_t H = (std::size_t)c.constant("CHANNELS_HEIGHT"), W = (std::size_t)c.constant("CHANNELS_WIDTH");
    if (c.weights.size() != O * C * H * W)
        throw std::runtime_error("exported cell " + c.identifier + ": " + std::to_string(c.weights.size()) + " weights, expected " + std::to_string(O * C * H * W));
    std::vector<std::int8_t> w(c.weights.size());
    for (std::size_t o = 0; o < O; ++o)
        for (std::size_t y = 0; y < H; ++y)
            for (std::size_t x = 0; x < W; ++x)
                for (std::size_t ch = 0; ch < C; ++ch)
                    w[o * C * H * W + (ch * H + y) * W + x] = c.weights[o * C * H * W + (y * W + x) * C + ch];
    auto cell = std::make_shared<FcCell>(c.identifier, (unsigned)O, exportedActivation(c));
    cell->setWeights(w);
    if (c.hasBiases) cell->setBiases(c.biases);
    cell->setQuantized(8);
    if (c.outputUnsigned >= 0) cell->setOutputUnsigned(c.outputUnsigned != 0);
    return cell;
}

inline std::shared_ptr<PoolCell> poolCellFromExport(const ExportedCell& c)
{
    auto it = c.names.find("POOLING");
    if (it == c.names.end() || (it->second != "Max" && it->second != "Average"))
        throw std::runtime_error("exported cell " + c.identifier + ": POOLING must be Max or Average");
    return std::make_shared<PoolCell>(c.identifier, std::vector<unsigned>{(unsigned)c.constant("POOL_WIDTH"), (unsigned)c.constant("POOL_HEIGHT")},
                                      (unsigned)c.constant("NB_OUTPUTS"),
                                      std::vector<unsigned>{(unsigned)c.constant("STRIDE_X"), (unsigned)c.constant("STRIDE_Y")},
                                      std::vector<unsigned>{(unsigned)c.constant("PADDING_X"), (unsigned)c.constant("PADDING_Y")},
                                      it->second == "Max" ? PoolCell::Max : PoolCell::Average);
}

inline std::shared_ptr<ElemWiseCell> elemWiseCellFromExport(const ExportedCell& c)
{
    auto it = c.names.find("ELEM_OP");
    if (it != c.names.end() && it->second != "Sum")
        throw std::runtime_error("exported cell " + c.identifier + ": only the Sum operation exists on the quantized path");
    auto cell = std::make_shared<ElemWiseCell>(c.identifier, (unsigned)c.constant("NB_OUTPUTS"), ElemWiseCell::Sum, exportedActivation(c));
    cell->setQuantized(8);
    if (c.outputUnsigned >= 0) cell->setOutputUnsigned(c.outputUnsigned != 0);
    return cell;
}

inline std::shared_ptr<ScalingCell> scalingCellFromExport(const ExportedCell& c)
{
    auto cell = std::make_shared<ScalingCell>(c.identifier, (unsigned)c.constant("NB_OUTPUTS"), c.scaling);
    cell->setQuantized(8);
    if (c.outputUnsigned >= 0) cell->setOutputUnsigned(c.outputUnsigned != 0);
    return cell;
}

}  // namespace N2D2
