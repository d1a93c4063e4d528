#!/usr/bin/env python3
"""Lists the devices and their properties (flow of samples/python/hello_query_device/hello_query_device.py)."""
import openvino_b200 as ov


def main() -> int:
    core = ov.Core()
    print("Available devices:")
    for device in core.available_devices:
        print(f"{device} :")
        print("\tSUPPORTED_PROPERTIES:")
        for key in core.get_property(device, "SUPPORTED_PROPERTIES"):
            if key in ("SUPPORTED_PROPERTIES",):
                continue
            try:
                value = core.get_property(device, key)
            except Exception as e:          # a write-only or context-dependent property
                value = f"UNSUPPORTED TYPE ({type(e).__name__})"
            print(f"\t\t{key}: {value}")
        print()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
