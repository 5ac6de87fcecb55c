/* TEST INFRASTRUCTURE ONLY.  Stand-in for the CANN platform query header: the
 * reference asks it for the number of vector cores. */
#ifndef ORACLE_REF_SHIM_PLATFORM_ASCENDC_H_
#define ORACLE_REF_SHIM_PLATFORM_ASCENDC_H_
#include <cstdint>
namespace platform_ascendc {
enum class CoreMemType { L0_A, L0_B, L0_C, L1, L2, UB, HBM };
class PlatformAscendCManager {
public:
    static PlatformAscendCManager* GetInstance() { return nullptr; }
    uint32_t GetCoreNumAiv() const { return 0; }
    uint32_t GetCoreNumAic() const { return 0; }
    uint64_t GetLibApiWorkSpaceSize() const { return 0; }
    void GetCoreMemSize(CoreMemType, uint64_t& size) const { size = 0; }
};
}  // namespace platform_ascendc
#endif
