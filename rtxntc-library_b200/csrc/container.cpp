#include "container.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>

#include "error.h"
#include "json_mini.h"
#include "network_shape.h"
#include "ntcb.h"

namespace ntcb
{

int LodToNeuralLod(int lod, int gridSizeScale, int neuralLods)
{
    // number of first colour mips that share latent mip 0, indexed by gridSizeScale - 1
    static const int sharedMips[6] = {2, 3, 3, 3, 4, 4};
    int neuralLod = (lod - sharedMips[gridSizeScale - 1] + 2) & ~1;
    return std::max(0, std::min(neuralLod, neuralLods - 2));
}

int GridDimension(int imageDimension, int neuralLod, int gridSizeScale)
{
    return std::max((imageDimension / gridSizeScale) >> neuralLod, 1);
}

int MakeGeometry(int width, int height, int channels, int mips, int gridSizeScale, int numFeatures, SetGeometry& out)
{
    if (width <= 0 || height <= 0 || channels <= 0 || mips <= 0)
    {
        SetError("Invalid TextureSetDesc: width (%d), height (%d), channels (%d) and mips (%d) must be positive numbers.",
            width, height, channels, mips);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (channels > kMaxChannels)
    {
        SetError("Invalid TextureSetDesc: too many channels (%d). Only up to %d channels are supported.", channels,
            kMaxChannels);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (mips > kMaxMips)
    {
        SetError("Invalid TextureSetDesc: too many mips (%d). Only up to %d mips are supported.", mips, kMaxMips);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (numFeatures <= 0 || numFeatures > 16 || (numFeatures % 4) != 0)
    {
        SetError("Invalid LatentShape: numFeatures (%d) must be a positive multiple of %d up to %d.", numFeatures, 4, 16);
        return NTCB_ERR_OUT_OF_RANGE;
    }
    if (gridSizeScale < 1 || gridSizeScale > 6)
    {
        SetError("Invalid LatentShape: gridSizeScale (%d) must be between 1 and 6.", gridSizeScale);
        return NTCB_ERR_OUT_OF_RANGE;
    }

    out = SetGeometry();
    out.width = width;
    out.height = height;
    out.channels = (channels + 1) & ~1;
    out.mips = mips;
    out.gridSizeScale = gridSizeScale;
    out.numFeatures = numFeatures;
    out.numLayers = (numFeatures + 3) / 4;

    const int minGridSize = int(float(std::min(width, height)) / float(gridSizeScale));
    int theoretical = 2;
    if (minGridSize >= 1)
        theoretical = std::max(2, int(1.f + std::floor(std::log2(float(minGridSize))))) & ~1;
    const int lastNeuralMip = LodToNeuralLod(mips - 1, gridSizeScale, kMaxNeuralMips);
    out.numNeuralMips = std::min(theoretical, lastNeuralMip + 2);

    uint64_t pixels = 0;
    for (int m = 0; m < out.numNeuralMips; ++m)
    {
        out.latentWidth[m] = GridDimension(width, m, gridSizeScale);
        out.latentHeight[m] = GridDimension(height, m, gridSizeScale);
        out.latentPixelOffset[m] = pixels;
        pixels += uint64_t(out.latentWidth[m]) * uint64_t(out.latentHeight[m]);
    }
    out.latentPixelOffset[out.numNeuralMips] = pixels;

    uint64_t texels = 0;
    for (int mip = 0; mip < mips; ++mip)
    {
        const int w = std::max(1, width >> mip), h = std::max(1, height >> mip);
        const int lod = LodToNeuralLod(mip, gridSizeScale, out.numNeuralMips);
        out.mipWidth[mip] = w;
        out.mipHeight[mip] = h;
        out.neuralLod[mip] = lod;
        const float widthScale = float(out.latentWidth[lod]) / float(w);
        const float heightScale = float(out.latentHeight[lod]) / float(h);
        out.positionScale[mip] = 0.5f * std::max(widthScale, heightScale);
        out.positionLod[mip] = std::max(-1.f, std::min(1.f, 0.25f * log2f(out.positionScale[mip])));
        out.mipTexelOffset[mip] = texels;
        texels += uint64_t(w) * uint64_t(h);
    }
    out.mipTexelOffset[mips] = texels;
    return NTCB_OK;
}

namespace
{

#pragma pack(push, 1)
struct FileHeader
{
    uint32_t signature;
    uint32_t version;
    uint64_t jsonChunkOffset;
    uint64_t jsonChunkSize;
    uint64_t binaryChunkOffset;
    uint64_t binaryChunkSize;
};
#pragma pack(pop)

constexpr uint32_t kSignature = 0x5845544E; // "NTEX"
constexpr uint32_t kVersion = 0x100;
constexpr uint64_t kSchemaVersion = 3;

struct View
{
    uint64_t offset = 0, storedSize = 0;
    bool compressed = false;
};

bool GetUnsigned(const json::Value& object, const char* name, bool required, uint64_t& out, const char* where)
{
    const json::Value* v = object.Find(name);
    if (!v)
    {
        if (required)
            SetError("%s: required field '%s' is missing.", where, name);
        return !required;
    }
    if (!v->IsUnsigned())
    {
        SetError("%s: field '%s' must be an unsigned integer.", where, name);
        return false;
    }
    out = v->integer;
    return true;
}

bool GetString(const json::Value& object, const char* name, std::string& out)
{
    const json::Value* v = object.Find(name);
    if (!v || v->kind != json::Kind::String)
        return false;
    out = v->text;
    return true;
}

const std::vector<json::Value>* GetArray(const json::Value& object, const char* name)
{
    static const std::vector<json::Value> empty;
    const json::Value* v = object.Find(name);
    if (!v)
        return &empty; // arrays are never required
    if (v->kind != json::Kind::Array)
        return nullptr;
    return &v->items;
}

struct Reader
{
    const uint8_t* binary;
    uint64_t binarySize;
    std::vector<View> views;

    // A view must exist, be uncompressed and hold at least `bytes`.
    int Fetch(uint64_t index, size_t bytes, void* dst, const char* what)
    {
        if (index >= views.size())
        {
            SetError("%s refers to buffer view %llu, but the file has only %zu views.", what, (unsigned long long)index,
                views.size());
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        const View& view = views[size_t(index)];
        if (view.compressed)
        {
            SetError("%s is stored with GDeflate compression, which this decoder does not read.", what);
            return NTCB_ERR_UNSUPPORTED;
        }
        if (view.storedSize < bytes)
        {
            SetError("%s: buffer view %llu holds %llu bytes, %zu are needed.", what, (unsigned long long)index,
                (unsigned long long)view.storedSize, bytes);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        memcpy(dst, binary + view.offset, bytes);
        return NTCB_OK;
    }

    // The whole of an optional view; `compressed` is set instead for a GDeflate view.
    int FetchWhole(uint64_t index, std::vector<uint8_t>& out, bool& compressed, uint64_t& offsetInBinaryChunk, uint64_t& storedSize,
        const char* what)
    {
        if (index >= views.size())
        {
            SetError("%s refers to buffer view %llu, but the file has only %zu views.", what, (unsigned long long)index,
                views.size());
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        const View& view = views[size_t(index)];
        compressed = view.compressed;
        offsetInBinaryChunk = view.offset;
        storedSize = view.storedSize;
        out.clear();
        if (!compressed)
            out.assign(binary + view.offset, binary + view.offset + view.storedSize);
        return NTCB_OK;
    }
};

// One MLP version of the document -> the row-major blob the reference keeps in memory
// (GenericInt8 or GenericFP8), smaller hidden layers zero-expanded.
int LoadNetwork(const json::Value& mlp, Reader& reader, std::vector<uint8_t>& int8Blob, std::vector<uint8_t>& fp8Blob)
{
    const std::vector<json::Value>* layers = GetArray(mlp, "layers");
    if (!layers)
    {
        SetError("MLP: 'layers' must be an array.");
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    if (layers->empty())
        return NTCB_OK;
    if (layers->size() != 4)
    {
        SetError("File describes an MLP with %d layers, while only %d layers are supported", int(layers->size()), 4);
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    std::string layout;
    if (GetString(mlp, "weightLayout", layout) && layout != "RowMajor")
    {
        SetError("Only row-major MLP weight layout is supported at this time.");
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }

    std::string weightType[4], scaleType[4], biasType[4];
    uint64_t inputs[4], outputs[4], weightView[4], scaleView[4], biasView[4];
    bool hasScaleView[4];
    for (int i = 0; i < 4; ++i)
    {
        const json::Value& layer = (*layers)[i];
        if (layer.kind != json::Kind::Object || !GetUnsigned(layer, "inputChannels", true, inputs[i], "MLPLayer") ||
            !GetUnsigned(layer, "outputChannels", true, outputs[i], "MLPLayer") ||
            !GetUnsigned(layer, "weightView", true, weightView[i], "MLPLayer") ||
            !GetUnsigned(layer, "biasView", true, biasView[i], "MLPLayer"))
            return NTCB_ERR_FILE_UNRECOGNIZED;
        hasScaleView[i] = layer.Find("scaleView") != nullptr;
        scaleView[i] = 0;
        if (hasScaleView[i] && !GetUnsigned(layer, "scaleView", true, scaleView[i], "MLPLayer"))
            return NTCB_ERR_FILE_UNRECOGNIZED;
        if (!GetString(layer, "weightType", weightType[i]) || !GetString(layer, "biasType", biasType[i]))
        {
            SetError("MLPLayer: 'weightType' and 'biasType' are required.");
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        GetString(layer, "scaleType", scaleType[i]);
    }

    bool isInt8 = true, isFp8 = true;
    for (int i = 0; i < 4; ++i)
    {
        isInt8 = isInt8 && weightType[i] == "Int8" && scaleType[i] == "Float32" && biasType[i] == "Int32";
        if (i < 3)
            isFp8 = isFp8 && weightType[i] == "FloatE4M3" && scaleType[i].empty() && biasType[i] == "Float16";
        else
            isFp8 = isFp8 && weightType[i] == "Int8" && scaleType[i] == "Float32" && biasType[i] == "Int32";
    }
    if (!isInt8 && !isFp8)
    {
        SetError("Only Int8 weights + Float32 scale + Int32 bias or FloatE4M3 + Float16 bias MLP configurations are "
                 "supported at this time.");
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    for (int i = 0; i < 4; ++i)
    {
        const bool smallerInputs = i > 0, smallerOutputs = i < 3;
        const bool inputsOk = smallerInputs ? inputs[i] <= uint64_t(kLayerInputs[i]) : inputs[i] == uint64_t(kLayerInputs[i]);
        const bool outputsOk = smallerOutputs ? outputs[i] <= uint64_t(kLayerOutputs[i]) : outputs[i] == uint64_t(kLayerOutputs[i]);
        if (!inputsOk || !outputsOk || inputs[i] == 0 || outputs[i] == 0)
        {
            SetError("File describes MLP layer %d with %d inputs and %d outputs, but that layer should have %s%d inputs "
                     "and %s%d outputs.",
                i, int(inputs[i]), int(outputs[i]), smallerInputs ? "at most " : "", kLayerInputs[i],
                smallerOutputs ? "at most " : "", kLayerOutputs[i]);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
    }

    std::vector<uint8_t>& blob = isInt8 ? int8Blob : fp8Blob;
    blob.assign(isInt8 ? kInt8BlobBytes : kFp8BlobBytes, 0);
    std::vector<uint8_t> temp;
    size_t weightOffset = 0;
    // offsets inside the blob (src/WeightLayout.cpp:228-255)
    size_t scaleOffset[4], biasOffset[4];
    if (isInt8)
    {
        size_t s = 8192, b = 8192 + 640;
        for (int i = 0; i < 4; ++i)
        {
            scaleOffset[i] = s;
            biasOffset[i] = b;
            s += 4u * kLayerOutputs[i];
            b += 4u * kLayerOutputs[i];
        }
    }
    else
    {
        size_t b = 8192;
        for (int i = 0; i < 3; ++i)
        {
            scaleOffset[i] = 0;
            biasOffset[i] = b;
            b += 2u * kLayerOutputs[i];
        }
        scaleOffset[3] = b;
        biasOffset[3] = b + 4u * 16;
    }

    for (int i = 0; i < 4; ++i)
    {
        const int nin = int(inputs[i]), nout = int(outputs[i]);
        temp.resize(size_t(nin) * nout);
        int rc = reader.Fetch(weightView[i], temp.size(), temp.data(), "MLP weight view");
        if (rc != NTCB_OK)
            return rc;
        // smaller layers land in the top-left corner of the full matrix (src/TextureSetMetadata.cpp:660-672)
        for (int n = 0; n < nout; ++n)
            memcpy(blob.data() + weightOffset + size_t(n) * kLayerInputs[i], temp.data() + size_t(n) * nin, size_t(nin));
        weightOffset += size_t(kLayerInputs[i]) * kLayerOutputs[i];

        const bool hasScale = isInt8 || i == 3;
        if (hasScale)
        {
            float* scales = reinterpret_cast<float*>(blob.data() + scaleOffset[i]);
            int provided = 0;
            if (hasScaleView[i])
            {
                rc = reader.Fetch(scaleView[i], 4u * nout, scales, "MLP scale view");
                if (rc != NTCB_OK)
                    return rc;
                provided = nout;
            }
            for (int n = provided; n < kLayerOutputs[i]; ++n)
                scales[n] = 1.0f; // src/TextureSetMetadata.cpp:733-742
        }
        const size_t biasElement = (isInt8 || i == 3) ? 4 : 2;
        rc = reader.Fetch(biasView[i], biasElement * nout, blob.data() + biasOffset[i], "MLP bias view");
        if (rc != NTCB_OK)
            return rc;
    }
    return NTCB_OK;
}

} // namespace

int LoadContainer(const void* data, size_t size, LoadedSet& out)
{
    out = LoadedSet();
    const uint8_t* bytes = static_cast<const uint8_t*>(data);
    if (!bytes)
    {
        SetError("The container pointer is NULL.");
        return NTCB_ERR_INVALID_ARGUMENT;
    }
    if (size < sizeof(FileHeader))
    {
        SetError("Failed to read the file header - file smaller than %zu bytes?", sizeof(FileHeader));
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    FileHeader header;
    memcpy(&header, bytes, sizeof header);
    if (header.signature != kSignature)
    {
        SetError("Unrecognized file format.");
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    if (header.version != kVersion)
    {
        SetError("Incompatible file format version: expected %d, got %d.", int(kVersion), int(header.version));
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    const uint64_t jsonEnd = header.jsonChunkOffset + header.jsonChunkSize;
    const uint64_t binaryEnd = header.binaryChunkOffset + header.binaryChunkSize;
    if (jsonEnd < header.jsonChunkOffset || binaryEnd < header.binaryChunkOffset || std::max(jsonEnd, binaryEnd) > size)
    {
        SetError("File incomplete: expected at least %llu bytes, actual size %zu bytes.",
            (unsigned long long)std::max(jsonEnd, binaryEnd), size);
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }

    json::Value document;
    std::string parseError;
    if (!json::Parse(reinterpret_cast<const char*>(bytes + header.jsonChunkOffset), size_t(header.jsonChunkSize), document,
            parseError) ||
        document.kind != json::Kind::Object)
    {
        SetError("The JSON chunk cannot be parsed: %s.", parseError.empty() ? "not an object" : parseError.c_str());
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }

    uint64_t schemaVersion = 0, width = 0, height = 0, numChannels = 0, numColorMips = 1;
    if (!GetUnsigned(document, "schemaVersion", true, schemaVersion, "Document"))
        return NTCB_ERR_FILE_UNRECOGNIZED;
    if (schemaVersion != kSchemaVersion)
    {
        SetError("Incompatible file schema version %u, expected %u", unsigned(schemaVersion), unsigned(kSchemaVersion));
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    if (!GetUnsigned(document, "width", true, width, "Document") || !GetUnsigned(document, "height", true, height, "Document") ||
        !GetUnsigned(document, "numChannels", true, numChannels, "Document") ||
        !GetUnsigned(document, "numColorMips", false, numColorMips, "Document"))
        return NTCB_ERR_FILE_UNRECOGNIZED;

    // buffer views (src/TextureSetMetadata.cpp:950-985)
    Reader reader;
    reader.binary = bytes + header.binaryChunkOffset;
    reader.binarySize = header.binaryChunkSize;
    const std::vector<json::Value>* views = GetArray(document, "views");
    if (!views)
    {
        SetError("Document: 'views' must be an array.");
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    for (size_t i = 0; i < views->size(); ++i)
    {
        const json::Value& v = (*views)[i];
        View view;
        if (v.kind != json::Kind::Object || !GetUnsigned(v, "offset", true, view.offset, "BufferView") ||
            !GetUnsigned(v, "storedSize", true, view.storedSize, "BufferView"))
            return NTCB_ERR_FILE_UNRECOGNIZED;
        std::string compression;
        if (GetString(v, "compression", compression) && compression != "None")
        {
            if (compression != "GDeflate")
            {
                SetError("Buffer view %zu has an unknown compression type '%s'.", i, compression.c_str());
                return NTCB_ERR_FILE_UNRECOGNIZED;
            }
            view.compressed = true;
        }
        if ((view.offset & 3) != 0)
        {
            SetError("Buffer view %zu has an offset (%llu) that is not a multiple of 4.", i, (unsigned long long)view.offset);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        if (view.offset + view.storedSize < view.offset || view.offset + view.storedSize > header.binaryChunkSize)
        {
            SetError("Buffer view %zu (offset %llu, size %llu) does not fit into the binary chunk (%llu bytes).", i,
                (unsigned long long)view.offset, (unsigned long long)view.storedSize,
                (unsigned long long)header.binaryChunkSize);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        reader.views.push_back(view);
    }

    // latent shape: numFeatures is stored, gridSizeScale is inferred from the first latent image
    // (src/TextureSetMetadata.cpp:1180-1208)
    const json::Value* latentShape = document.Find("latentShape");
    const std::vector<json::Value>* latents = GetArray(document, "latents");
    if (!latentShape || latentShape->kind != json::Kind::Object || !latents || latents->empty())
    {
        SetError("The file holds no latent data; it cannot be decompressed.");
        return NTCB_ERR_FILE_INCOMPATIBLE;
    }
    uint64_t numFeatures = 0;
    if (!GetUnsigned(*latentShape, "numFeatures", true, numFeatures, "LatentShape"))
        return NTCB_ERR_FILE_UNRECOGNIZED;
    struct LatentImage
    {
        uint64_t width = 0, height = 0;
        std::vector<uint64_t> layerViews;
    };
    std::vector<LatentImage> images;
    for (const json::Value& entry : *latents)
    {
        LatentImage image;
        if (entry.kind != json::Kind::Object || !GetUnsigned(entry, "width", true, image.width, "LatentImage") ||
            !GetUnsigned(entry, "height", true, image.height, "LatentImage"))
            return NTCB_ERR_FILE_UNRECOGNIZED;
        const std::vector<json::Value>* layerViews = GetArray(entry, "layerViews");
        if (!layerViews)
        {
            SetError("LatentImage: 'layerViews' must be an array.");
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        for (const json::Value& index : *layerViews)
        {
            if (!index.IsUnsigned())
            {
                SetError("LatentImage: 'layerViews' must hold unsigned integers.");
                return NTCB_ERR_FILE_UNRECOGNIZED;
            }
            image.layerViews.push_back(index.integer);
        }
        images.push_back(std::move(image));
    }
    if (width > 0x7FFFFFFF || height > 0x7FFFFFFF || numChannels > 0x7FFFFFFF || numColorMips > 0x7FFFFFFF ||
        numFeatures > 0x7FFFFFFF)
    {
        SetError("Invalid TextureSetDesc: values out of range.");
        return NTCB_ERR_OUT_OF_RANGE;
    }
    const float widthRatio = float(width) / float(std::max<uint64_t>(images[0].width, 1));
    const float heightRatio = float(height) / float(std::max<uint64_t>(images[0].height, 1));
    const int gridSizeScale = int(roundf(std::min(widthRatio, heightRatio)));

    SetGeometry& geo = out.geometry;
    int rc = MakeGeometry(int(width), int(height), int(numChannels), int(numColorMips), gridSizeScale, int(numFeatures), geo);
    if (rc != NTCB_OK)
        return rc;

    // the decoder relies on the library's own latent geometry (src/TextureSet.cpp:164-196)
    if (int(images.size()) < geo.numNeuralMips)
    {
        SetError("The file holds %zu latent images, %d are needed.", images.size(), geo.numNeuralMips);
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    for (int m = 0; m < geo.numNeuralMips; ++m)
    {
        if (images[m].width != uint64_t(geo.latentWidth[m]) || images[m].height != uint64_t(geo.latentHeight[m]))
        {
            SetError("Neural MIP %d dimensions (%dx%d) don't match the expected dimensions (%dx%d)", m, int(images[m].width),
                int(images[m].height), geo.latentWidth[m], geo.latentHeight[m]);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        if (int(images[m].layerViews.size()) != geo.numLayers)
        {
            SetError("Latent image %d has %zu layer views, %d are expected.", m, images[m].layerViews.size(), geo.numLayers);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
    }
    const std::vector<json::Value>* colorMips = GetArray(document, "colorMips");
    if (!colorMips || int(colorMips->size()) < geo.mips)
    {
        SetError("The file describes %zu color mips, %d are needed.", colorMips ? colorMips->size() : size_t(0), geo.mips);
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    for (int mip = 0; mip < geo.mips; ++mip)
    {
        const json::Value& entry = (*colorMips)[mip];
        uint64_t latentMip = 0;
        if (entry.kind != json::Kind::Object || !entry.Find("latentMip") ||
            !GetUnsigned(entry, "latentMip", true, latentMip, "ColorMip") || !entry.Find("positionLod") ||
            !entry.Find("positionScale"))
        {
            SetError("Color MIP %d must specify latentMip, positionLod and positionScale.", mip);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        if (int(latentMip) != geo.neuralLod[mip])
        {
            SetError("Color MIP %d specifies latent image index %d, but it is expected to be %d.", mip, int(latentMip),
                geo.neuralLod[mip]);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        // positionScale / positionLod are recomputed from the geometry, as the reference's CUDA path
        // does (src/TextureSet.cpp:450-463); the stored values only serve the graphics path.
    }

    // channel headers: the colour space each channel was stored in (src/TextureSetMetadata.cpp:479-495)
    for (int c = 0; c < kMaxChannels; ++c)
        out.channelColorSpaces[c] = 0;
    const std::vector<json::Value>* channelHeaders = GetArray(document, "channels");
    if (channelHeaders && !channelHeaders->empty())
    {
        if (channelHeaders->size() != size_t(numChannels) && channelHeaders->size() != size_t(geo.channels))
        {
            SetError("The file describes %d texture channels while %d are expected", int(channelHeaders->size()), geo.channels);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        for (size_t c = 0; c < channelHeaders->size(); ++c)
        {
            const json::Value& entry = (*channelHeaders)[c];
            std::string space;
            if (entry.kind != json::Kind::Object)
            {
                SetError("Document: 'channels' must hold objects.");
                return NTCB_ERR_FILE_UNRECOGNIZED;
            }
            if (!GetString(entry, "colorSpace", space) || space == "Linear")
                out.channelColorSpaces[c] = 0;
            else if (space == "sRGB")
                out.channelColorSpaces[c] = 1;
            else if (space == "HLG")
                out.channelColorSpaces[c] = 2;
            else
            {
                SetError("Channel %zu has an unknown color space '%s'.", c, space.c_str());
                return NTCB_ERR_FILE_UNRECOGNIZED;
            }
        }
    }

    // texture headers (src/JsonFileFormat.cpp:118-127, src/TextureSetMetadata.cpp:460-468)
    out.textures.clear();
    const std::vector<json::Value>* textureHeaders = GetArray(document, "textures");
    if (!textureHeaders)
    {
        SetError("Document: 'textures' must be an array.");
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    for (size_t t = 0; t < textureHeaders->size(); ++t)
    {
        const json::Value& entry = (*textureHeaders)[t];
        if (entry.kind != json::Kind::Object)
        {
            SetError("Document: 'textures' must hold objects.");
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        LoadedTexture texture;
        uint64_t first = 0, count = 0;
        if (!GetString(entry, "name", texture.name))
        {
            SetError("Texture %zu: required field 'name' is missing.", t);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        if (!GetUnsigned(entry, "firstChannel", true, first, "Texture") || !GetUnsigned(entry, "numChannels", true, count, "Texture"))
            return NTCB_ERR_FILE_UNRECOGNIZED;
        texture.firstChannel = int(first);
        texture.numChannels = int(count);
        struct EnumField
        {
            const char* name;
            int* target;
            std::vector<const char*> values; // the index is the enum's value
        };
        const EnumField enums[] = {
            {"channelFormat", &texture.channelFormat, {"UNKNOWN", "UNORM8", "UNORM16", "FLOAT16", "FLOAT32", "UINT32"}},
            {"rgbColorSpace", &texture.rgbColorSpace, {"Linear", "sRGB", "HLG"}},
            {"alphaColorSpace", &texture.alphaColorSpace, {"Linear", "sRGB", "HLG"}},
            {"bcFormat", &texture.blockCompressedFormat, {"None", "BC1", "BC2", "BC3", "BC4", "BC5", "BC6", "BC7"}},
        };
        for (const EnumField& field : enums)
        {
            std::string text;
            if (!GetString(entry, field.name, text))
                continue; // optional: the default stays
            int value = -1;
            for (size_t v = 0; v < field.values.size(); ++v)
                if (text == field.values[v])
                    value = int(v);
            if (value < 0)
            {
                SetError("Texture %zu: field '%s' has an unknown value '%s'.", t, field.name, text.c_str());
                return NTCB_ERR_FILE_UNRECOGNIZED;
            }
            *field.target = value;
        }
        texture.modeBuffers.assign(size_t(geo.mips), std::vector<uint8_t>());
        texture.modeBufferCompressed.assign(size_t(geo.mips), 0);
        texture.modeBufferOffset.assign(size_t(geo.mips), 0);
        texture.modeBufferStoredSize.assign(size_t(geo.mips), 0);
        const std::vector<json::Value>* modeBuffers = GetArray(entry, "bcModeBuffers");
        if (!modeBuffers)
        {
            SetError("Texture %zu: 'bcModeBuffers' must be an array.", t);
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        for (const json::Value& item : *modeBuffers)
            {
                uint64_t mipLevel = 0, view = 0;
                if (item.kind != json::Kind::Object)
                {
                    SetError("Texture %zu: 'bcModeBuffers' must hold objects.", t);
                    return NTCB_ERR_FILE_UNRECOGNIZED;
                }
                if (!GetUnsigned(item, "mipLevel", true, mipLevel, "BCModeBuffer") || !GetUnsigned(item, "view", true, view, "BCModeBuffer"))
                    return NTCB_ERR_FILE_UNRECOGNIZED;
                std::vector<uint8_t> bytes;
                bool compressed = false;
                uint64_t offsetInChunk = 0, storedSize = 0;
                rc = reader.FetchWhole(view, bytes, compressed, offsetInChunk, storedSize, "BC7 mode buffer");
                if (rc != NTCB_OK)
                    return rc;
                if (mipLevel >= uint64_t(geo.mips))
                    continue; // as the reference: an entry for a mip the set does not have is dropped
                texture.modeBuffers[size_t(mipLevel)] = std::move(bytes);
                texture.modeBufferCompressed[size_t(mipLevel)] = compressed ? 1 : 0;
                texture.modeBufferOffset[size_t(mipLevel)] = uint64_t(reader.binary - static_cast<const uint8_t*>(data)) + offsetInChunk;
                texture.modeBufferStoredSize[size_t(mipLevel)] = storedSize;
            }
        out.textures.push_back(texture);
    }

    // latent planes -> device order
    out.latents.resize(size_t(geo.TotalLatentPixels()) * geo.numLayers);
    for (int m = 0; m < geo.numNeuralMips; ++m)
    {
        const size_t plane = size_t(geo.latentWidth[m]) * geo.latentHeight[m];
        for (int layer = 0; layer < geo.numLayers; ++layer)
        {
            uint16_t* dst = out.latents.data() + size_t(geo.latentPixelOffset[m]) * geo.numLayers + plane * layer;
            rc = reader.Fetch(images[m].layerViews[layer], plane * 2, dst, "Latent image view");
            if (rc != NTCB_OK)
                return rc;
        }
    }

    // networks
    const std::vector<json::Value>* mlpVersions = GetArray(document, "mlpVersions");
    if (!mlpVersions)
    {
        SetError("Document: 'mlpVersions' must be an array.");
        return NTCB_ERR_FILE_UNRECOGNIZED;
    }
    for (const json::Value& mlp : *mlpVersions)
    {
        if (mlp.kind != json::Kind::Object)
        {
            SetError("Document: 'mlpVersions' must hold objects.");
            return NTCB_ERR_FILE_UNRECOGNIZED;
        }
        rc = LoadNetwork(mlp, reader, out.int8Blob, out.fp8Blob);
        if (rc != NTCB_OK)
            return rc;
    }
    if (out.int8Blob.empty() && out.fp8Blob.empty())
    {
        SetError("The file holds no MLP weights; it cannot be decompressed.");
        return NTCB_ERR_FILE_INCOMPATIBLE;
    }
    ClearError();
    return NTCB_OK;
}

} // namespace ntcb
