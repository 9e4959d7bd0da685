// CPU emulation of one warp of the dequant-GEMV kernel: 32 host threads play the lanes, the MMA and the
// shared-memory loads are emulated (slai_b200/csrc/gemv_formats.cuh), everything else is the kernel's own
// source.  Usage: host_emul <fmt> <K> <blocks.bin (16 rows, GGUF order)> <v.bin (K f32)>  -> prints 16 floats;
// with a fifth argument NV (2, 4 or 8) v.bin holds NV vectors, the batched per-lane code runs and NV x 16 floats are printed.
// Compiled for the host only; it never touches a GPU.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <pthread.h>
#include <cuda_fp16.h>

#include "../slai_b200/csrc/gemv_formats.cuh"
#include "../slai_b200/csrc/layout.cuh"

namespace hostemu {
thread_local int lane;
thread_local Warp* warp;
}  // namespace hostemu

using namespace gemvfmt;

struct Job {
    int fmt, K, nsteps;
    uint32_t tile0;  // shared-space address of the tile's first tile-step block
    int step_bytes;
    Smem S;
    hostemu::Warp* W;
    float acc[32][2];
    int nv = 0;            // > 0: batched code against nv staged vectors
    uint32_t vstride = 0;  // bytes between the staged vectors (digits and sums alike)
    float bacc[32][8][2];
};

template <class F>
static void lane_body(Job* J, int lane) {
    LaneCtx L;
    lane_init<F>(L, lane, J->S);
    float a = 0.f, b = 0.f;
    for (int s = 0; s < J->nsteps; s++) F::compute(J->tile0 + (uint32_t)s * J->step_bytes, s, L, J->S, a, b);
    J->acc[lane][0] = a;
    J->acc[lane][1] = b;
}

template <class F, int NV>
static void lane_body_batch(Job* J, int lane) {
    LaneCtx L;
    lane_init<F>(L, lane, J->S);
    const uint32_t bvs = L.bmul ? J->vstride : 0u;
    float a[NV], b[NV];
    for (int v = 0; v < NV; v++) a[v] = b[v] = 0.f;
    for (int s = 0; s < J->nsteps; s++) F::template compute_batch<NV>(J->tile0 + (uint32_t)s * J->step_bytes, s, L, J->S, bvs, J->vstride, a, b);
    for (int v = 0; v < NV; v++) {
        J->bacc[lane][v][0] = a[v];
        J->bacc[lane][v][1] = b[v];
    }
}
template <class F>
static void lane_dispatch(Job* J, int lane) {
    switch (J->nv) {
        case 0: lane_body<F>(J, lane); break;
        case 2: lane_body_batch<F, 2>(J, lane); break;
        case 4: lane_body_batch<F, 4>(J, lane); break;
        case 8: lane_body_batch<F, 8>(J, lane); break;
    }
}

struct ThreadArg { Job* J; int lane; };
static void* thread_main(void* p) {
    ThreadArg* A = (ThreadArg*)p;
    hostemu::lane = A->lane;
    hostemu::warp = A->J->W;
    switch (A->J->fmt) {
        case 12: lane_dispatch<Q4K>(A->J, A->lane); break;
        case 13: lane_dispatch<Q5K>(A->J, A->lane); break;
        case 14: lane_dispatch<Q6K>(A->J, A->lane); break;
        case 8: lane_dispatch<Q80>(A->J, A->lane); break;
    }
    return nullptr;
}

static std::vector<uint8_t> read_file(const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) { perror(path); exit(2); }
    fseek(f, 0, SEEK_END);
    long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    std::vector<uint8_t> d(n);
    if (fread(d.data(), 1, n, f) != (size_t)n) exit(2);
    fclose(f);
    return d;
}

int main(int argc, char** argv) {
    if (argc < 5) return 2;
    const int fmt = atoi(argv[1]), K = atoi(argv[2]);
    std::vector<uint8_t> raw = read_file(argv[3]);
    std::vector<uint8_t> vb = read_file(argv[4]);
    const float* vall = (const float*)vb.data();
    const int nv = argc > 5 ? atoi(argv[5]) : 0;
    const int nvec = nv > 0 ? nv : 1;
    if (nv != 0 && nv != 2 && nv != 4 && nv != 8) return 2;
    const int be = fmt == 8 ? 32 : 256, bb = fmt == 8 ? 34 : fmt == 12 ? 144 : fmt == 13 ? 176 : 210;
    const int nbk = K / be;
    if ((int)raw.size() != 16 * nbk * bb || (int)vb.size() != 4 * K * nvec) { fprintf(stderr, "size mismatch\n"); return 2; }

    // device layout: one tile of 16 rows, tile-major (layout.cuh)
    const int sbytes = layout::step_bytes(fmt);
    const int nsteps = (int)layout::num_steps(fmt, K);
    std::vector<uint8_t> tile((size_t)nsteps * sbytes, 0);
    for (int r = 0; r < 16; r++)
        for (int b = 0; b < nbk; b++) layout::place_block(fmt, raw.data() + ((size_t)r * nbk + b) * bb, tile.data(), r, b, K);

    // staging (mirrors the kernels' staging with no prologue): power-of-two scale, integer rounding, four base-256
    // digit planes, per-sub-block digit sums; one region per vector, `vstride` bytes apart
    const int Kp = (K + 255) & ~255;
    const int sv_gran = (fmt == 12 || fmt == 13) ? 32 : fmt == 14 ? 16 : 0;
    const size_t sv_bytes = sv_gran ? (size_t)(Kp / sv_gran) * 16 : 0;
    const int plane = Kp + 32;
    const size_t dig0 = ZERO_BYTES;
    const size_t sv0 = dig0 + 4 * (size_t)plane;
    const size_t vstride = (4 * (size_t)plane + sv_bytes + 15) & ~(size_t)15;
    const size_t tile_off = (size_t)(dig0 + nvec * vstride + 127) & ~(size_t)127;
    std::vector<unsigned char> smem(tile_off + tile.size() + 64, 0);
    memcpy(smem.data() + tile_off, tile.data(), tile.size());
    std::vector<float> scales(nvec, 1.f);
    for (int vi = 0; vi < nvec; vi++) {
        const float* v = vall + (size_t)vi * K;
        const size_t d0 = dig0 + vi * vstride, s0 = sv0 + vi * vstride;
        float mx = 0.f;
        for (int k = 0; k < K; k++) mx = fmaxf(mx, fabsf(v[k]));
        float scale = 1.f;
        if (mx > 0.f) { int e; frexpf(mx, &e); if (e < -90) e = -90; scale = ldexpf(1.0f, 26 - e); }
        scales[vi] = scale;
        std::vector<int> sums(sv_gran ? (size_t)(Kp / sv_gran) * 4 : 0, 0);
        for (int k = 0; k < Kp; k++) {
            const float x = k < K ? v[k] * scale : 0.f;
            const uint32_t word = frag::digits_word((int)nearbyintf(x));
            for (int p = 0; p < 4; p++) {
                const int d = (int)(signed char)((word >> (8 * p)) & 0xFF);
                smem[d0 + (size_t)p * plane + k] = (unsigned char)(d & 0xFF);
                if (sv_gran) sums[(k / sv_gran) * 4 + p] += d;
            }
        }
        if (sv_gran == 16) {  // Q6_K: 4 x s32 per sub-block
            memcpy(smem.data() + s0, sums.data(), sums.size() * 4);
        } else if (sv_gran == 32) {  // Q4_K / Q5_K: byte table (two base-128 digits per sum), see gemv_formats.cuh
            for (int J = 0; J < Kp / 32; J++)
                for (int q = 0; q < 4; q++) {
                    const int sd = sums[J * 4 + q], hi = (sd + 64) >> 7, lo = sd - hi * 128;
                    unsigned char* tab = smem.data() + s0 + (size_t)(J >> 3) * 128;
                    tab[(2 * q) * 16 + (J & 7)] = (unsigned char)(hi & 0xFF);
                    tab[(2 * q + 1) * 16 + (J & 7)] = (unsigned char)(lo & 0xFF);
                }
        }
    }

    hostemu::Warp W;
    pthread_barrier_init(&W.bar, nullptr, 32);
    W.smem = smem.data();
    Job J;
    J.fmt = fmt; J.K = K; J.W = &W;
    J.nsteps = nsteps; J.tile0 = (uint32_t)tile_off; J.step_bytes = sbytes;
    J.S.zero = 0; J.S.dig = (uint32_t)dig0; J.S.plane = plane; J.S.sv = (uint32_t)sv0;
    J.nv = nv; J.vstride = (uint32_t)vstride;
    pthread_t th[32];
    ThreadArg args[32];
    for (int l = 0; l < 32; l++) { args[l] = {&J, l}; pthread_create(&th[l], nullptr, thread_main, &args[l]); }
    for (int l = 0; l < 32; l++) pthread_join(th[l], nullptr);
    for (int vi = 0; vi < nvec; vi++)
        for (int r = 0; r < 16; r++) {
            const int g = r & 7, which = r >> 3;
            auto acc = [&](int l) { return nv ? J.bacc[l][vi][which] : J.acc[l][which]; };
            // xor-1 then xor-2 shuffle reduction as in the kernel
            const float a0 = acc(g * 4 + 0) + acc(g * 4 + 1);
            const float a1 = acc(g * 4 + 2) + acc(g * 4 + 3);
            printf("%.9g\n", (a0 + a1) / scales[vi]);
        }
    return 0;
}
