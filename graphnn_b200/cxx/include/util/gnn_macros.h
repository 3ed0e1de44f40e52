// Tokens, enums and error macros of the graphnn operator interface
// (the names of include/util/gnn_macros.h:16-213 in the reference), so that driver code
// written against the reference compiles against this library.
#ifndef S2V_GNN_MACROS_H
#define S2V_GNN_MACROS_H

#include <cstddef>
#include <cstdio>
#include <exception>
#include <iostream>
#include <stdexcept>
#include <string>

namespace gnn
{

typedef unsigned int uint;

enum class MatType { dense, sparse, row_sparse };
enum class PropErr { N = 0, T = 1 };
enum class Trans { N = 0, T = 1 };
enum class MatMode { cpu = 0, gpu = 1 };
enum class Phase { TRAIN = 0, TEST = 1 };
enum class EleType { FLOAT32 = 0, FLOAT64 = 1, INT32 = 2, UNKNOWN = 3 };

struct CPU { static const MatMode type = MatMode::cpu; };
struct GPU { static const MatMode type = MatMode::gpu; };
struct DENSE { static const MatType type = MatType::dense; };
struct CSR_SPARSE { static const MatType type = MatType::sparse; };
struct ROW_SPARSE { static const MatType type = MatType::row_sparse; };

template <typename Dtype> inline EleType Dtype2Enum() { return EleType::UNKNOWN; }
template <> inline EleType Dtype2Enum<float>() { return EleType::FLOAT32; }
template <> inline EleType Dtype2Enum<double>() { return EleType::FLOAT64; }
template <> inline EleType Dtype2Enum<int>() { return EleType::INT32; }

// Same contract as the reference: print the failed condition and terminate.
#define ASSERT(condition, message)                                                                   \
    do {                                                                                             \
        if (!(condition)) {                                                                          \
            std::cerr << "Assertion `" #condition "` failed in " << __FILE__ << " line " << __LINE__ \
                      << ": " << message << std::endl;                                               \
            std::terminate();                                                                        \
        }                                                                                            \
    } while (false)

#define NOT_IMPLEMENTED                                                                               \
    {                                                                                                 \
        throw std::logic_error(std::string("not implemented virtual func: ") + std::string(__FUNCTION__)); \
    }

#define MAT_TYPE_SWITCH(type, matType, ...)              \
    switch (type) {                                      \
        case MatType::dense: {                           \
            typedef DENSE matType;                       \
            { __VA_ARGS__ }                              \
        } break;                                         \
        case MatType::sparse: {                          \
            typedef CSR_SPARSE matType;                  \
            { __VA_ARGS__ }                              \
        } break;                                         \
        default:                                         \
            throw std::logic_error("unknown type");      \
    }

}  // namespace gnn
#endif
