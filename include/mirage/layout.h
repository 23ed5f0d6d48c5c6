// Device- and shared-memory layout tags (reference: include/mirage/layout.h:22-58).
// DmemLayout decides how float-mode loaders address a tensor's last two dims;
// fingerprint mode indexes row-major whatever the tag says.  SmemLayout is
// accepted for drop-in compatibility; the executor picks its own staging layout
// (TMA swizzle) and results never depend on it.
#pragma once
namespace mirage {
namespace layout {
enum DmemLayout { DmemRowMajor = 100, DmemColumnMajor = 101, DmemUnknownLayout = 199 };
enum SmemLayout { SmemRowMajor = 200, SmemColumnMajor = 201,
                  SmemRowMajorTensorOpMultiplicand_Crosswise16 = 202,
                  SmemRowMajorTensorOpMultiplicand_Crosswise32 = 203,
                  SmemRowMajorTensorOpMultiplicand_Crosswise64 = 204,
                  SmemColumnMajorTensorOpMultiplicand_Crosswise16 = 205,
                  SmemColumnMajorTensorOpMultiplicand_Crosswise32 = 206,
                  SmemColumnMajorTensorOpMultiplicand_Crosswise64 = 207, SmemUnknownLayout = 299 };
char const *to_string(DmemLayout l);
char const *to_string(SmemLayout l);
} // namespace layout
} // namespace mirage
