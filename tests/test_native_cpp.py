"""Runs the C++ unit tests of the native API (tests/cpp/native_api_test.cpp): the file is
compiled against the package's headers, linked to the in-tree ``_comms.so`` and driven
through one C entry point.  Mirrors the reference's GoogleTest unit level
(comms/torchcomms/tests/unit/cpp) without needing GoogleTest."""
import ctypes
import os
import subprocess
import sysconfig

import torch  # noqa: F401  (loads libtorch before the test library)


def test_native_cpp_api(tmp_path):
    from torch.utils.cpp_extension import include_paths

    import torchcomms_b200  # noqa: F401  (loads _comms.so)

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "torchcomms_b200")
    lib = tmp_path / "libnative_api_test.so"
    cmd = ["/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++", "-shared", "-fPIC", "-std=c++17", "-O1",
           "-D_GLIBCXX_USE_CXX11_ABI=1", "-I", os.path.join(pkg, "csrc")]
    for inc in include_paths(device_type="cuda") + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]:
        cmd += ["-isystem", inc]
    cmd += [os.path.join(root, "tests", "cpp", "native_api_test.cpp"), "-o", str(lib), "-L", pkg, "-l:_comms.so",
            f"-Wl,-rpath,{pkg}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    dll = ctypes.CDLL(str(lib))
    dll.b200c_run_native_tests.restype = ctypes.c_int
    dll.b200c_run_native_tests.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
    message = ctypes.create_string_buffer(8192)
    failures = dll.b200c_run_native_tests(str(tmp_path).encode(), message, len(message))
    assert failures == 0, message.value.decode()
