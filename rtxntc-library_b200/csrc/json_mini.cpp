#include "json_mini.h"

#include <cerrno>
#include <cstdlib>
#include <cstring>

namespace ntcb::json
{

const Value* Value::Find(const char* name) const
{
    if (kind != Kind::Object)
        return nullptr;
    for (auto const& member : members)
        if (member.first == name)
            return &member.second;
    return nullptr;
}

namespace
{

struct Parser
{
    const char* p;
    const char* end;
    std::string& error;
    int depth = 0;

    bool Fail(const char* message)
    {
        if (error.empty())
            error = message;
        return false;
    }

    void SkipSpace()
    {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r'))
            ++p;
    }

    bool Literal(const char* word)
    {
        size_t n = strlen(word);
        if (size_t(end - p) < n || memcmp(p, word, n) != 0)
            return Fail("invalid literal");
        p += n;
        return true;
    }

    bool ParseString(std::string& out)
    {
        if (p >= end || *p != '"')
            return Fail("expected a string");
        ++p;
        out.clear();
        while (p < end && *p != '"')
        {
            char c = *p++;
            if (c == '\\')
            {
                if (p >= end)
                    return Fail("unterminated escape");
                char e = *p++;
                switch (e)
                {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u':
                {
                    if (end - p < 4)
                        return Fail("truncated \\u escape");
                    unsigned code = 0;
                    for (int i = 0; i < 4; ++i)
                    {
                        char h = *p++;
                        code <<= 4;
                        if (h >= '0' && h <= '9') code |= unsigned(h - '0');
                        else if (h >= 'a' && h <= 'f') code |= unsigned(h - 'a' + 10);
                        else if (h >= 'A' && h <= 'F') code |= unsigned(h - 'A' + 10);
                        else return Fail("invalid \\u escape");
                    }
                    // names and enum values in NTC documents are ASCII; encode the rest as UTF-8
                    if (code < 0x80) out.push_back(char(code));
                    else if (code < 0x800)
                    {
                        out.push_back(char(0xC0 | (code >> 6)));
                        out.push_back(char(0x80 | (code & 0x3F)));
                    }
                    else
                    {
                        out.push_back(char(0xE0 | (code >> 12)));
                        out.push_back(char(0x80 | ((code >> 6) & 0x3F)));
                        out.push_back(char(0x80 | (code & 0x3F)));
                    }
                    break;
                }
                default: return Fail("invalid escape");
                }
            }
            else
                out.push_back(c);
        }
        if (p >= end)
            return Fail("unterminated string");
        ++p;
        return true;
    }

    bool ParseNumber(Value& out)
    {
        const char* start = p;
        bool negative = false, integer = true;
        if (p < end && *p == '-') { negative = true; ++p; }
        const char* digits = p;
        while (p < end && *p >= '0' && *p <= '9') ++p;
        if (p == digits)
            return Fail("invalid number");
        if (p < end && *p == '.')
        {
            integer = false;
            ++p;
            while (p < end && *p >= '0' && *p <= '9') ++p;
        }
        if (p < end && (*p == 'e' || *p == 'E'))
        {
            integer = false;
            ++p;
            if (p < end && (*p == '+' || *p == '-')) ++p;
            while (p < end && *p >= '0' && *p <= '9') ++p;
        }
        std::string literal(start, p);
        out.kind = Kind::Number;
        out.number = strtod(literal.c_str(), nullptr);
        out.isInteger = integer;
        out.negative = negative;
        if (integer && !negative)
        {
            errno = 0;
            out.integer = strtoull(literal.c_str(), nullptr, 10);
            if (errno != 0)
                return Fail("integer out of range");
        }
        return true;
    }

    bool ParseValue(Value& out)
    {
        if (++depth > 64)
            return Fail("document nested too deeply");
        SkipSpace();
        if (p >= end)
            return Fail("unexpected end of document");
        bool ok = true;
        char c = *p;
        if (c == '{')
        {
            ++p;
            out.kind = Kind::Object;
            SkipSpace();
            if (p < end && *p == '}') { ++p; }
            else
            {
                for (;;)
                {
                    SkipSpace();
                    std::string name;
                    if (!ParseString(name)) { ok = false; break; }
                    SkipSpace();
                    if (p >= end || *p != ':') { ok = Fail("expected ':'"); break; }
                    ++p;
                    out.members.emplace_back(std::move(name), Value());
                    if (!ParseValue(out.members.back().second)) { ok = false; break; }
                    SkipSpace();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == '}') { ++p; break; }
                    ok = Fail("expected ',' or '}'");
                    break;
                }
            }
        }
        else if (c == '[')
        {
            ++p;
            out.kind = Kind::Array;
            SkipSpace();
            if (p < end && *p == ']') { ++p; }
            else
            {
                for (;;)
                {
                    out.items.emplace_back();
                    if (!ParseValue(out.items.back())) { ok = false; break; }
                    SkipSpace();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == ']') { ++p; break; }
                    ok = Fail("expected ',' or ']'");
                    break;
                }
            }
        }
        else if (c == '"')
        {
            out.kind = Kind::String;
            ok = ParseString(out.text);
        }
        else if (c == 't') { ok = Literal("true"); out.kind = Kind::Bool; out.boolean = true; }
        else if (c == 'f') { ok = Literal("false"); out.kind = Kind::Bool; out.boolean = false; }
        else if (c == 'n') { ok = Literal("null"); out.kind = Kind::Null; }
        else
            ok = ParseNumber(out);
        --depth;
        return ok;
    }
};

} // namespace

bool Parse(const char* text, size_t length, Value& out, std::string& error)
{
    error.clear();
    // the chunk is stored with a terminating NUL (and possibly padding); stop at the first NUL
    size_t n = 0;
    while (n < length && text[n] != '\0')
        ++n;
    Parser parser{text, text + n, error};
    out = Value();
    if (!parser.ParseValue(out))
        return false;
    parser.SkipSpace();
    if (parser.p != parser.end)
    {
        error = "trailing characters after the document";
        return false;
    }
    return true;
}

} // namespace ntcb::json
