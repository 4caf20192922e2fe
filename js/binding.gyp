{
  # node-gyp build of the N-API addon (js/binding.cc).  The addon is pure marshalling: all device
  # code lives in tfjs-core_b200/libtfjs_cuda.so, built by tfjs-core_b200/build.py with nvcc for
  # sm_100a, which this target links against and finds at run time next to itself.
  "targets": [{
    "target_name": "tfjs_cuda",
    "sources": ["binding.cc"],
    "include_dirs": ["../include"],
    "defines": ["NAPI_VERSION=6"],
    "cflags_cc": ["-std=c++14", "-O2", "-Wall"],
    "libraries": [
      "-L<(module_root_dir)/../tfjs-core_b200", "-ltfjs_cuda",
      "-Wl,-rpath,'$$ORIGIN/../../../tfjs-core_b200'"
    ]
  }]
}
