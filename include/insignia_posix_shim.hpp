// Lets the reference's Windows console drivers build on Linux unchanged: force-include this header
// (`nvcc -include insignia_posix_shim.hpp driver.cu`).  It supplies main() in terms of the driver's
// wmain(int, wchar_t**) and the two wide-character CRT calls the drivers use (_wfopen, _wtoi).
#pragma once
#include <clocale>
#include <cstdio>
#include <cstdlib>
#include <cwchar>
#include <string>
#include <vector>

int wmain(int argc, wchar_t **argv);

inline std::string insignia_narrow(const wchar_t *w)
{
    std::string out;
    for (; w && *w; ++w) { // UTF-8 encode; arguments came from UTF-8 in main() below
        const unsigned long c = static_cast<unsigned long>(*w);
        if (c < 0x80) out += char(c);
        else if (c < 0x800) { out += char(0xc0 | (c >> 6)); out += char(0x80 | (c & 0x3f)); }
        else if (c < 0x10000) { out += char(0xe0 | (c >> 12)); out += char(0x80 | ((c >> 6) & 0x3f)); out += char(0x80 | (c & 0x3f)); }
        else { out += char(0xf0 | (c >> 18)); out += char(0x80 | ((c >> 12) & 0x3f)); out += char(0x80 | ((c >> 6) & 0x3f)); out += char(0x80 | (c & 0x3f)); }
    }
    return out;
}

inline FILE *_wfopen(const wchar_t *path, const wchar_t *mode)
{
    return std::fopen(insignia_narrow(path).c_str(), insignia_narrow(mode).c_str());
}

inline int _wtoi(const wchar_t *s) { return int(std::wcstol(s, nullptr, 10)); }

int main(int argc, char **argv)
{
    std::vector<std::wstring> wide(static_cast<size_t>(argc));
    std::vector<wchar_t *> ptr(static_cast<size_t>(argc) + 1, nullptr);
    for (int i = 0; i < argc; i++) {
        const unsigned char *s = reinterpret_cast<const unsigned char *>(argv[i]);
        while (*s) { // UTF-8 decode (malformed bytes pass through as themselves)
            unsigned long c = *s++;
            int more = c >= 0xf0 ? 3 : c >= 0xe0 ? 2 : c >= 0xc0 ? 1 : 0;
            if (more) c &= (0x3f >> more);
            while (more-- && (*s & 0xc0) == 0x80) c = (c << 6) | (*s++ & 0x3f);
            wide[size_t(i)] += wchar_t(c);
        }
        ptr[size_t(i)] = wide[size_t(i)].data();
    }
    return wmain(argc, ptr.data());
}
