#!/bin/bash
# Builds the reference's NVIDIA library (unmodified sources: torch class flash_comm_t + NVSHMEM
# kernels) for sm_100a into baseline/_ref/nv_build/libflash.so with a hand-written nvcc line.
# The reference's own CMake project cannot configure offline: it asks for an NVSHMEM CMake package
# (find_package(NVSHMEM), nvidia/CMakeLists.txt:21) and targets sm_90a only (:8). The NVSHMEM
# headers, device archive and host library come from the nvidia-nvshmem wheel in site-packages.
# Needs no GPU. Loading the result needs the CUDA driver (libcuda.so.1), i.e. a GPU box.
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
REF=${1:-$HERE/../../reference}/nvidia
OUT="$HERE/_ref/nv_build"
PY=${PYTHON:-python}
NVSH=$($PY -c "import nvidia.nvshmem, os; print(os.path.dirname(nvidia.nvshmem.__path__[0] + '/'))" 2>/dev/null || true)
[ -d "$NVSH/include" ] || NVSH=$($PY -c "import sysconfig, os; print(os.path.join(sysconfig.get_paths()['purelib'], 'nvidia', 'nvshmem'))")
TORCH_INC=$($PY -c "import torch.utils.cpp_extension as c; print(' '.join('-I' + p for p in c.include_paths()))" 2>/dev/null)
TORCH_LIB=$($PY -c "import torch, os; print(os.path.join(os.path.dirname(torch.__file__), 'lib'))" 2>/dev/null)
PY_INC=$($PY -c "import sysconfig; print('-I' + sysconfig.get_paths()['include'])")
CUDA=${CUDA_HOME:-/usr/local/cuda}
mkdir -p "$OUT"
cd "$OUT"
INC="-I$REF/src/include -I$REF -I$NVSH/include -I$CUDA/include"
nvcc -gencode arch=compute_100a,code=sm_100a -rdc=true -std=c++17 -O2 -w -Xcompiler -fPIC $INC \
     -c "$REF/src/fast_alltoall/flash_alltoall_nvshmem.cu" -o flash_alltoall_nvshmem.o
for f in alltoall_algorithm alltoall_global_scheduler alltoall_local_scheduler alltoall_matrix; do
  g++ -O2 -std=c++17 -w -fPIC $INC -c "$REF/src/fast_alltoall/$f.cc" -o $f.o
done
g++ -O2 -std=c++17 -w -fPIC -D_GLIBCXX_USE_CXX11_ABI=1 $INC $TORCH_INC $PY_INC -c "$REF/alltoall_nvshmem.cpp" -o alltoall_nvshmem.o
nvcc -gencode arch=compute_100a,code=sm_100a -dlink -Xcompiler -fPIC flash_alltoall_nvshmem.o -L"$NVSH/lib" -lnvshmem_device -o dlink.o
ln -sf "$NVSH/lib/libnvshmem_host.so.3" libnvshmem_host.so
STUBS=""
[ -e "$CUDA/lib64/stubs/libcuda.so" ] && STUBS="-L$CUDA/lib64/stubs"
g++ -shared -o libflash.so alltoall_nvshmem.o alltoall_algorithm.o alltoall_global_scheduler.o alltoall_local_scheduler.o alltoall_matrix.o \
    flash_alltoall_nvshmem.o dlink.o -L"$NVSH/lib" -lnvshmem_device -L. -lnvshmem_host -L"$TORCH_LIB" -lc10 -ltorch -ltorch_cpu -lc10_cuda \
    -ltorch_cuda -L"$CUDA/lib64" $STUBS -lcudart -lcudadevrt -lcuda -Wl,-rpath,"$NVSH/lib" -Wl,-rpath,"$TORCH_LIB"
rm -f ./*.o
echo "$OUT/libflash.so"
