// Device-to-device copy of 256 MiB by differently shaped kernels, against cudaMemcpyAsync: the
// measurement behind the shape of k_copy_stream (src/kernels/dispatch.cu), the single-rank
// AllReduce. Device-timed with CUDA events, three buffer pairs in rotation (each larger than
// L2), median and minimum of 15 runs.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o bench/copy_variants bench/copy_variants.cu
//   ./bench/copy_variants
//
// Variants: v0 one contiguous share per 512-thread CTA; v1 grid-stride tiles of U 16-byte
// vectors per thread, with or without cache hints (ld.global.nc.L1::no_allocate, st.global.cs);
// v2 256-bit accesses; v3 / v4 bulk-async copies (cp.async.bulk) through shared memory with one
// issuing thread per CTA; v5 one tile per CTA; v6 64 contiguous bytes per thread.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <vector>
#include <algorithm>
#define CK(x) do{cudaError_t e_=(x); if(e_!=cudaSuccess){printf("ERR %s line %d\n",cudaGetErrorString(e_),__LINE__); return 1;}}while(0)

__device__ __forceinline__ uint4 ldnc(const void* p){uint4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];":"=r"(v.x),"=r"(v.y),"=r"(v.z),"=r"(v.w):"l"(p)); return v;}
__device__ __forceinline__ void stcs(void* p, uint4 v){asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"::"l"(p),"r"(v.x),"r"(v.y),"r"(v.z),"r"(v.w):"memory");}

// V0: contiguous share per CTA, 8 in flight
__global__ void __launch_bounds__(512) v0(char* dst,const char* src,size_t bytes,size_t share){
  size_t lo=size_t(blockIdx.x)*share; if(lo>=bytes) return; size_t n=min(share,bytes-lo); dst+=lo; src+=lo;
  size_t nv=n>>4; size_t t=threadIdx.x, nt=blockDim.x; size_t i=t;
  for(;i+7*nt<nv;i+=8*nt){uint4 r[8];
#pragma unroll
    for(int u=0;u<8;++u) r[u]=*reinterpret_cast<const uint4*>(src+((i+u*nt)<<4));
#pragma unroll
    for(int u=0;u<8;++u) *reinterpret_cast<uint4*>(dst+((i+u*nt)<<4))=r[u];}
  for(;i<nv;i+=nt) *reinterpret_cast<uint4*>(dst+(i<<4))=*reinterpret_cast<const uint4*>(src+(i<<4));
}
// V1: grid-stride tiles, U x 16B per thread, nc + cs
template<int U,bool HINT>
__global__ void v1(char* dst,const char* src,size_t bytes){
  size_t nv=bytes>>4; size_t nt=blockDim.x; size_t tile=nt*U;
  for(size_t base=size_t(blockIdx.x)*tile; base<nv; base+=size_t(gridDim.x)*tile){
    uint4 r[U];
#pragma unroll
    for(int u=0;u<U;++u){size_t i=base+u*nt+threadIdx.x; if(i<nv) r[u]= HINT? ldnc(src+(i<<4)) : *reinterpret_cast<const uint4*>(src+(i<<4));}
#pragma unroll
    for(int u=0;u<U;++u){size_t i=base+u*nt+threadIdx.x; if(i<nv){ if(HINT) stcs(dst+(i<<4),r[u]); else *reinterpret_cast<uint4*>(dst+(i<<4))=r[u];}}
  }
}
// V5: one tile per CTA, no loop
template<int U,bool HINT>
__global__ void v5(char* dst,const char* src,size_t bytes){
  size_t nv=bytes>>4; size_t nt=blockDim.x; size_t base=size_t(blockIdx.x)*nt*U;
  uint4 r[U];
#pragma unroll
  for(int u=0;u<U;++u){size_t i=base+u*nt+threadIdx.x; if(i<nv) r[u]= HINT? ldnc(src+(i<<4)) : *reinterpret_cast<const uint4*>(src+(i<<4));}
#pragma unroll
  for(int u=0;u<U;++u){size_t i=base+u*nt+threadIdx.x; if(i<nv){ if(HINT) stcs(dst+(i<<4),r[u]); else *reinterpret_cast<uint4*>(dst+(i<<4))=r[u];}}
}
// V6: per-thread contiguous 64B (4x16B adjacent) - warp covers 2 KiB contiguous
template<bool HINT>
__global__ void v6(char* dst,const char* src,size_t bytes){
  size_t n64=bytes>>6; size_t i=size_t(blockIdx.x)*blockDim.x+threadIdx.x; size_t stride=size_t(gridDim.x)*blockDim.x;
  for(;i<n64;i+=stride){ uint4 r[4];
#pragma unroll
    for(int u=0;u<4;++u) r[u]=HINT? ldnc(src+(i<<6)+u*16) : *reinterpret_cast<const uint4*>(src+(i<<6)+u*16);
#pragma unroll
    for(int u=0;u<4;++u){ if(HINT) stcs(dst+(i<<6)+u*16,r[u]); else *reinterpret_cast<uint4*>(dst+(i<<6)+u*16)=r[u]; }
  }
}
// V2: 256-bit loads/stores
struct alignas(32) u8v{unsigned v[8];};
__device__ __forceinline__ u8v ld32(const void* p){u8v r; asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];":"=r"(r.v[0]),"=r"(r.v[1]),"=r"(r.v[2]),"=r"(r.v[3]),"=r"(r.v[4]),"=r"(r.v[5]),"=r"(r.v[6]),"=r"(r.v[7]):"l"(p)); return r;}
__device__ __forceinline__ void st32(void* p,const u8v& r){asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"::"l"(p),"r"(r.v[0]),"r"(r.v[1]),"r"(r.v[2]),"r"(r.v[3]),"r"(r.v[4]),"r"(r.v[5]),"r"(r.v[6]),"r"(r.v[7]):"memory");}
template<int U>
__global__ void v2(char* dst,const char* src,size_t bytes){
  size_t nv=bytes>>5; size_t nt=blockDim.x; size_t tile=nt*U;
  for(size_t base=size_t(blockIdx.x)*tile; base<nv; base+=size_t(gridDim.x)*tile){
    u8v r[U];
#pragma unroll
    for(int u=0;u<U;++u){size_t i=base+u*nt+threadIdx.x; if(i<nv) r[u]=ld32(src+(i<<5));}
#pragma unroll
    for(int u=0;u<U;++u){size_t i=base+u*nt+threadIdx.x; if(i<nv) st32(dst+(i<<5),r[u]);}
  }
}
// V3: bulk async copy through shared memory, one issuing thread per CTA
__device__ __forceinline__ unsigned smem_u32(const void* p){return (unsigned)__cvta_generic_to_shared(p);}
template<int STAGES>
__global__ void v3(char* dst,const char* src,size_t bytes,unsigned chunk){
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bar[STAGES];
  if(threadIdx.x!=0) return;
  for(int s=0;s<STAGES;++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;"::"r"(smem_u32(&bar[s])));
  asm volatile("fence.mbarrier_init.release.cluster;":::"memory");
  const size_t nchunks=(bytes+chunk-1)/chunk;
  // chunks of this CTA: blockIdx.x, +gridDim.x, ...
  size_t mine = nchunks>blockIdx.x ? (nchunks-blockIdx.x+gridDim.x-1)/gridDim.x : 0;
  auto issue_load=[&](size_t k){ size_t c=blockIdx.x+k*gridDim.x; size_t off=c*chunk; unsigned len=(unsigned)min((size_t)chunk,bytes-off); int s=k%STAGES;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"::"r"(smem_u32(&bar[s])),"r"(len):"memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"::"r"(smem_u32(smem+size_t(s)*chunk)),"l"(src+off),"r"(len),"r"(smem_u32(&bar[s])):"memory"); };
  size_t issued=0;
  for(;issued<mine && issued<(size_t)STAGES;++issued) issue_load(issued);
  for(size_t k=0;k<mine;++k){
    int s=k%STAGES; unsigned phase=(k/STAGES)&1;
    unsigned done=0; unsigned spins=0;
    while(!done){ asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0,1,0,p;\n}":"=r"(done):"r"(smem_u32(&bar[s])),"r"(phase):"memory"); if(++spins>(1u<<20)) return; }
    size_t c=blockIdx.x+k*gridDim.x; size_t off=c*chunk; unsigned len=(unsigned)min((size_t)chunk,bytes-off);
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"::"l"(dst+off),"r"(smem_u32(smem+size_t(s)*chunk)),"r"(len):"memory");
    asm volatile("cp.async.bulk.commit_group;":::"memory");
    // refill: stage of chunk k+1-STAGES... we refill stage s for chunk k+STAGES once its store has read smem
    if(k+STAGES<mine){
      // allow at most STAGES-1 ... wait until the store of chunk k has read its smem: simplest wait_group.read 0 would serialize; instead lag by one
      asm volatile("cp.async.bulk.wait_group.read 0;":::"memory");
      issue_load(k+STAGES);
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;":::"memory");
}
// V4: like V3 but refills lag (keeps L stores outstanding before reusing a stage)
template<int STAGES,int LAG>
__global__ void v4(char* dst,const char* src,size_t bytes,unsigned chunk){
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) unsigned long long bar[STAGES];
  if(threadIdx.x!=0) return;
  for(int s=0;s<STAGES;++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;"::"r"(smem_u32(&bar[s])));
  asm volatile("fence.mbarrier_init.release.cluster;":::"memory");
  const size_t nchunks=(bytes+chunk-1)/chunk;
  size_t mine = nchunks>blockIdx.x ? (nchunks-blockIdx.x+gridDim.x-1)/gridDim.x : 0;
  auto issue_load=[&](size_t k){ size_t c=blockIdx.x+k*gridDim.x; size_t off=c*chunk; unsigned len=(unsigned)min((size_t)chunk,bytes-off); int s=k%STAGES;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"::"r"(smem_u32(&bar[s])),"r"(len):"memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"::"r"(smem_u32(smem+size_t(s)*chunk)),"l"(src+off),"r"(len),"r"(smem_u32(&bar[s])):"memory"); };
  // loads run STAGES-LAG ahead of stores; before loading chunk j into its stage, the store of chunk j-STAGES must have read smem:
  // stores committed so far = k+1 when we are at chunk k; store j-STAGES done reading when outstanding <= (k - (j-STAGES))
  size_t issued=0;
  for(;issued<mine && issued<(size_t)(STAGES-LAG);++issued) issue_load(issued);
  for(size_t k=0;k<mine;++k){
    int s=k%STAGES; unsigned phase=(k/STAGES)&1;
    unsigned done=0; unsigned spins=0;
    while(!done){ asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0,1,0,p;\n}":"=r"(done):"r"(smem_u32(&bar[s])),"r"(phase):"memory"); if(++spins>(1u<<20)) return; }
    size_t c=blockIdx.x+k*gridDim.x; size_t off=c*chunk; unsigned len=(unsigned)min((size_t)chunk,bytes-off);
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"::"l"(dst+off),"r"(smem_u32(smem+size_t(s)*chunk)),"r"(len):"memory");
    asm volatile("cp.async.bulk.commit_group;":::"memory");
    if(issued<mine){
      // chunk `issued` goes to stage issued%STAGES, last used by chunk issued-STAGES (if any), whose store is k-(issued-STAGES) groups back
      // issued = k+STAGES-LAG  => that store is LAG groups back: allow LAG-? outstanding
      asm volatile("cp.async.bulk.wait_group.read %0;"::"n"(LAG):"memory");
      issue_load(issued); ++issued;
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;":::"memory");
}

int main(){
  const size_t bytes=256u<<20;
  char *a[3],*b[3];
  for(int i=0;i<3;++i){CK(cudaMalloc(&a[i],bytes)); CK(cudaMalloc(&b[i],bytes)); CK(cudaMemset(a[i],i+1,bytes)); CK(cudaMemset(b[i],0,bytes));}
  cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  int sms=148; cudaDeviceGetAttribute(&sms,cudaDevAttrMultiProcessorCount,0);
  auto run=[&](const char* name, auto fn)->int{
    for(int w=0;w<3;++w) fn(b[w%3],a[w%3]);
    CK(cudaDeviceSynchronize());
    std::vector<float> ts;
    for(int it=0;it<15;++it){ cudaEventRecord(e0); fn(b[it%3],a[it%3]); cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); float ms; cudaEventElapsedTime(&ms,e0,e1); ts.push_back(ms);}    
    CK(cudaGetLastError());
    std::sort(ts.begin(),ts.end());
    // verify
    unsigned char h[64]; CK(cudaMemcpy(h,b[2]+bytes-64,64,cudaMemcpyDeviceToHost)); bool ok=true; for(int i=0;i<64;++i) ok&=h[i]==3;
    CK(cudaMemset(b[2],0,bytes));
    printf("%-28s median %.4f ms  min %.4f  algbw %.1f GB/s  %s\n",name,ts[ts.size()/2],ts[0],bytes/ts[ts.size()/2]/1e6,ok?"ok":"BAD"); fflush(stdout); return 0;};
  run("cudaMemcpyAsync",[&](char*d,char*s){cudaMemcpyAsync(d,s,bytes,cudaMemcpyDeviceToDevice,0);});
  for(int rep=0;rep<2;++rep){
  for(int per: {8,12,16,24,32,48}){ char nm[64];
    snprintf(nm,64,"v1 U4 hint 256thr x%d/SM",per); run(nm,[&](char*d,char*s){v1<4,true><<<sms*per,256>>>(d,s,bytes);});
    snprintf(nm,64,"v1 U2 hint 256thr x%d/SM",per); run(nm,[&](char*d,char*s){v1<2,true><<<sms*per,256>>>(d,s,bytes);});
  }
  for(int per: {8,16,32}){ char nm[64];
    snprintf(nm,64,"v1 U4 hint 128thr x%d/SM",per); run(nm,[&](char*d,char*s){v1<4,true><<<sms*per,128>>>(d,s,bytes);});
    snprintf(nm,64,"v2 256bit U2 256thr x%d/SM",per); run(nm,[&](char*d,char*s){v2<2><<<sms*per,256>>>(d,s,bytes);});
    snprintf(nm,64,"v2 256bit U1 256thr x%d/SM",per); run(nm,[&](char*d,char*s){v2<1><<<sms*per,256>>>(d,s,bytes);});
    snprintf(nm,64,"v6 64B/thr hint 256thr x%d/SM",per); run(nm,[&](char*d,char*s){v6<true><<<sms*per,256>>>(d,s,bytes);});
  }
  {size_t nv=bytes>>4; 
   run("v5 tile U4 hint 256thr",[&](char*d,char*s){v5<4,true><<<(unsigned)((nv+256*4-1)/(256*4)),256>>>(d,s,bytes);});
   run("v5 tile U8 hint 256thr",[&](char*d,char*s){v5<8,true><<<(unsigned)((nv+256*8-1)/(256*8)),256>>>(d,s,bytes);});
   run("v5 tile U4 nohint 256thr",[&](char*d,char*s){v5<4,false><<<(unsigned)((nv+256*4-1)/(256*4)),256>>>(d,s,bytes);});
   run("v5 tile U4 hint 512thr",[&](char*d,char*s){v5<4,true><<<(unsigned)((nv+512*4-1)/(512*4)),512>>>(d,s,bytes);});
   run("v5 tile U2 hint 256thr",[&](char*d,char*s){v5<2,true><<<(unsigned)((nv+256*2-1)/(256*2)),256>>>(d,s,bytes);});
   run("v5 tile U16 hint 256thr",[&](char*d,char*s){v5<16,true><<<(unsigned)((nv+256*16-1)/(256*16)),256>>>(d,s,bytes);});}
  run("cudaMemcpyAsync",[&](char*d,char*s){cudaMemcpyAsync(d,s,bytes,cudaMemcpyDeviceToDevice,0);});
  }
  printf("done\n");
  return 0;
}
