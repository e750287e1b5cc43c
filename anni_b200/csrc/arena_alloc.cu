/*
** Device memory for the optimizer's flats with the GPU's memory compression switched on.
**
** The reference's optimizer owns its flats (lang/lm_adam.c:217-311 allocates them with
** gpu_malloc), so where they live is this library's business.  B200 can keep an allocation
** "compressible": the L2 then writes lines that compress well (a zeroed gradient, above all)
** back to HBM at a fraction of their size.  Such memory comes from the driver's virtual
** memory interface, not from cudaMalloc: a physical allocation with the compression flag,
** mapped into a reserved address range.  The driver entry points are looked up through
** the runtime (cudaGetDriverEntryPoint), so the library does not link against libcuda and
** still loads on a machine without a driver.
**
** When the device or the driver does not offer compression, the calls say so and the
** caller uses plain memory; nothing here changes results, only how many bytes cross HBM.
*/
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>
#include <mutex>
#include "optstep_internal.h"

namespace {

struct driver_api {
	CUresult (*GetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
	CUresult (*Create)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
	CUresult (*Release)(CUmemGenericAllocationHandle);
	CUresult (*AddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
	CUresult (*AddressFree)(CUdeviceptr, size_t);
	CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
	CUresult (*Unmap)(CUdeviceptr, size_t);
	CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
	CUresult (*GetPropsFromHandle)(CUmemAllocationProp *, CUmemGenericAllocationHandle);
	bool ok;
};

driver_api g_drv;
std::once_flag g_drv_once;

template <typename F> bool lookup(const char *name, F *fn)
{
	void *p = NULL;
	cudaDriverEntryPointQueryResult st;

	if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &st) != cudaSuccess
	    || st != cudaDriverEntryPointSuccess || !p) {
		(void)cudaGetLastError();
		return false;
	}
	*fn = reinterpret_cast<F>(p);
	return true;
}

void load_driver(void)
{
	g_drv.ok = lookup("cuMemGetAllocationGranularity", &g_drv.GetAllocationGranularity)
	    && lookup("cuMemCreate", &g_drv.Create) && lookup("cuMemRelease", &g_drv.Release)
	    && lookup("cuMemAddressReserve", &g_drv.AddressReserve)
	    && lookup("cuMemAddressFree", &g_drv.AddressFree) && lookup("cuMemMap", &g_drv.Map)
	    && lookup("cuMemUnmap", &g_drv.Unmap) && lookup("cuMemSetAccess", &g_drv.SetAccess)
	    && lookup("cuMemGetAllocationPropertiesFromHandle", &g_drv.GetPropsFromHandle);
}

}	/* namespace */

/*
** nbytes of zeroed device memory on the current device, compressible if the device grants
** it.  *mapped_bytes is the size to hand back to anni_arena_free; *compressed says whether
** the driver really made the allocation compressible.  ANNI_E_LIMIT: compression is not
** available here (nothing was allocated; use cudaMalloc).
*/
extern "C" int anni_arena_alloc(size_t nbytes, void **out, size_t *mapped_bytes, int *compressed)
{
	CUmemAllocationProp prop;
	CUmemAllocationProp got;
	CUmemAccessDesc acc;
	CUmemGenericAllocationHandle handle;
	CUdeviceptr ptr = 0;
	size_t gran = 0;
	size_t size;
	int dev = 0;

	if (!out || !mapped_bytes || nbytes == 0)
		return ANNI_E_ARG;
	*out = NULL;
	*mapped_bytes = 0;
	if (compressed)
		*compressed = 0;
	if (cudaFree(0) != cudaSuccess || cudaGetDevice(&dev) != cudaSuccess)
		return ANNI_E_CUDA;
	std::call_once(g_drv_once, load_driver);
	if (!g_drv.ok)
		return ANNI_E_LIMIT;
	memset(&prop, 0, sizeof(prop));
	prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
	prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
	prop.location.id = dev;
	prop.allocFlags.compressionType = CU_MEM_ALLOCATION_COMP_GENERIC;
	if (g_drv.GetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS
	    || gran == 0)
		return ANNI_E_LIMIT;
	size = (nbytes + gran - 1) / gran * gran;
	if (g_drv.Create(&handle, size, &prop, 0) != CUDA_SUCCESS)
		return ANNI_E_LIMIT;
	memset(&got, 0, sizeof(got));
	if (g_drv.GetPropsFromHandle(&got, handle) != CUDA_SUCCESS
	    || got.allocFlags.compressionType != CU_MEM_ALLOCATION_COMP_GENERIC) {
		g_drv.Release(handle);		/* the driver fell back to plain memory: not what was asked for */
		return ANNI_E_LIMIT;
	}
	if (g_drv.AddressReserve(&ptr, size, 0, 0, 0) != CUDA_SUCCESS) {
		g_drv.Release(handle);
		return ANNI_E_NOMEM;
	}
	memset(&acc, 0, sizeof(acc));
	acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
	acc.location.id = dev;
	acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
	if (g_drv.Map(ptr, size, 0, handle, 0) != CUDA_SUCCESS) {
		g_drv.AddressFree(ptr, size);
		g_drv.Release(handle);
		return ANNI_E_NOMEM;
	}
	g_drv.Release(handle);		/* the mapping keeps the memory alive until it is unmapped */
	if (g_drv.SetAccess(ptr, size, &acc, 1) != CUDA_SUCCESS
	    || cudaMemset((void *)ptr, 0, size) != cudaSuccess) {
		g_drv.Unmap(ptr, size);
		g_drv.AddressFree(ptr, size);
		return ANNI_E_CUDA;
	}
	*out = (void *)ptr;
	*mapped_bytes = size;
	if (compressed)
		*compressed = 1;
	return ANNI_OK;
}

extern "C" int anni_arena_free(void *ptr, size_t mapped_bytes)
{
	if (!ptr)
		return ANNI_OK;
	std::call_once(g_drv_once, load_driver);
	if (!g_drv.ok || mapped_bytes == 0)
		return ANNI_E_ARG;
	if (cudaDeviceSynchronize() != cudaSuccess)
		return ANNI_E_CUDA;
	if (g_drv.Unmap((CUdeviceptr)ptr, mapped_bytes) != CUDA_SUCCESS
	    || g_drv.AddressFree((CUdeviceptr)ptr, mapped_bytes) != CUDA_SUCCESS)
		return ANNI_E_CUDA;
	return ANNI_OK;
}
