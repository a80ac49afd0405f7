// A small JSON reader for the document chunk of NTC containers: objects, arrays, numbers, strings,
// booleans and null, parsed into a tree.  The container's schema (field names and which are
// required) is applied by the loader in container.cpp; unknown fields are simply never asked for,
// which is how the reference's schema-driven reader treats them (src/JsonSerialization.cpp:850-868).
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace ntcb::json
{

enum class Kind
{
    Null,
    Bool,
    Number,
    String,
    Array,
    Object
};

struct Value
{
    Kind kind = Kind::Null;
    bool boolean = false;
    double number = 0.0;
    bool isInteger = false; // the literal had no fraction or exponent
    uint64_t integer = 0;   // valid when isInteger and the literal was not negative
    bool negative = false;
    std::string text;
    std::vector<Value> items;                            // Array
    std::vector<std::pair<std::string, Value>> members;  // Object, in document order

    const Value* Find(const char* name) const;
    bool IsUnsigned() const { return kind == Kind::Number && isInteger && !negative; }
};

// Parses `length` bytes of UTF-8 JSON.  On failure returns false and describes the problem.
bool Parse(const char* text, size_t length, Value& out, std::string& error);

} // namespace ntcb::json
