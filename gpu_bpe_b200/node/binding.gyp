{
  "targets": [{
    "target_name": "b200bpe",
    "sources": ["addon.cc"],
    "include_dirs": ["../../include"],
    "libraries": ["-L<(module_root_dir)/..", "-lb200bpe", "-Wl,-rpath,<(module_root_dir)/.."],
    "cflags_cc": ["-std=c++17"],
    "defines": ["NAPI_VERSION=8"]
  }]
}
