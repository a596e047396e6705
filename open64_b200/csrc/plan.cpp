// Tile-plan chooser: the B200 counterpart of the reference's tile decision
// (LOOP_MODEL::Model, osprey/be/lno/model.cxx:540, scored by Evaluate :1289 as
// cycles = max(resource, latency); cache blocking from Cache_Model,
// osprey/be/lno/cache_model.cxx:6483).  Pure host code, no CUDA calls.
//
// The search space is what the kernels are instantiated for: tile_m = 128, tile_n in
// {256, 128}, one CTA or a pair of CTAs per tile; each candidate is scored with a two-resource model (tensor pipe vs. the
// shared-memory fill rate) times the number of waves over the persistent grid.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "umma_gemm.cuh"

namespace o64 {

// Machine parameters (the reference keeps issue rate / register count / cache geometry here:
// osprey/be/lno/model.cxx:739-743, osprey/common/com/x8664/config_cache_targ.cxx:80-420).
static const double kClockGHz = 1.5;            // sustained SM clock under load, approx.
static const double kDenseBf16FlopPerClkSm = 8192.0;
static const double kSmemFillBytesPerClkSm = 96.0;  // L2 -> shared memory through TMA, approx.
static const double kLoadLatencyClk = 1900.0;        // TMA issue -> data in shared memory -> barrier, measured ~1.3 us

static int elem_bytes(int kind) { return kind == O64_KIND_BF16 ? 2 : (kind == O64_KIND_F32 ? 4 : 1); }

// The K split of a last, partly filled wave of tiles (CTA-pair kernels): `tiles` tiles of `kb` K
// blocks on `pairs` CTA pairs.  Whole tiles take (tiles / pairs + 1) * kb K-block times; with the
// tiles of the last wave cut along K over the pairs it is tiles / pairs whole tiles, one piece, and
// the hand-over (a partial accumulator stored, published, read back and added: measured at about 24
// K-block times of the 256-row kernel).  Pieces stay at least a sixth of a tile long (at most seven pieces per tile) and the split
// must save 8 % to be taken.  Returns the K-block times per pair; *tail_tiles = 0: whole tiles.
long long tail_model(long long tiles, int pairs, long long kb, int rows_per_cta, long long max_pairs_by_memory,
                     int force, int *tail_tiles, int *tail_pairs) {
    *tail_tiles = 0;
    *tail_pairs = 0;
    if (pairs < 1) pairs = 1;
    const long long rem = tiles % pairs, full = tiles / pairs;
    const long long whole = (full + (rem ? 1 : 0)) * kb;
    // the 512-row kernel keeps whole tiles: both of its accumulators fill tensor memory, its epilogue is
    // exposed, and the extra registers of the hand-over cost its ordinary epilogue more than the split saves
    if (rem == 0 || pairs < 2 || force == 0 || rows_per_cta == 256) return whole;
    long long min_share = (kb + 5) / 6;
    if (min_share < 4) min_share = 4;
    long long sp = pairs;
    if (rem * kb / sp < min_share) sp = rem * kb / min_share;
    if (sp > max_pairs_by_memory) sp = max_pairs_by_memory;
    if (sp <= rem) return whole;  // pieces as long as whole tiles: nothing to gain
    const long long share = (rem * kb + sp - 1) / sp;
    const long long handover = 24;
    const long long cut = full * kb + share + handover;
    if (force != 1 && cut * 100 > whole * 92) return whole;
    *tail_tiles = (int)rem;
    *tail_pairs = (int)sp;
    return cut;
}

// cta_group = 1: a CTA owns a 128 x tile_n tile.  cta_group = 2: a pair of CTAs owns a
// tile_m x tile_n tile (tile_m = 256: 128 rows per CTA; tile_m = 512: 256 rows per CTA as two
// accumulators issued by two threads); each CTA loads its rows of A and tile_n / 2 rows of B
// per K block.
static double predict_ms(int kind, int epi, int64_t M, int64_t N, int64_t K, int tile_n, int num_ctas,
                         int cta_group, int tile_m) {
    const int eb = elem_bytes(kind);
    const int block_k = 128 / eb;
    const int out_n = (epi == EPI_SWIGLU) ? tile_n / 2 : tile_n;
    const int rows_per_cta = tile_m / cta_group;
    const int units = num_ctas / cta_group;  // CTAs or CTA pairs working side by side
    const double tiles = double((M + tile_m - 1) / tile_m) * double((N + out_n - 1) / out_n);
    double waves = double(int64_t((tiles + units - 1) / units));
    const double kblocks = double((K + block_k - 1) / block_k);
    if (cta_group == 2 && units >= 2) {
        // a partly filled last wave may be cut along K (umma_common.cuh, work_item)
        int tt = 0, tp = 0;
        const long long t = tail_model((long long)tiles, units, (long long)kblocks, rows_per_cta, kTailMaxPairs, -1, &tt, &tp);
        // measured on M x 8192 x 8192 (M = 129 ... 1024): about a third of the K-block times the split
        // saves on paper come back as time - with every SM busy the chip, which runs these kernels at
        // its power limit, clocks lower - so a shape is not chosen for the full paper gain
        if (tt > 0) waves -= 0.35 * (waves - double(t) / kblocks);
    }
    const double flop_rate = kDenseBf16FlopPerClkSm * (eb == 1 ? 2.0 : 1.0);
    // measured: a tcgen05.mma of 128 rows costs about the same whether N is 128 or 256; paired
    // MMAs chained on one accumulator run about a tenth slower than alternated between two
    const double n_eff = tile_n < 256 ? 256.0 : double(tile_n);
    const double issue = (rows_per_cta == 256) ? 1.0 : (cta_group == 2 ? 1.10 : 1.02);
    double mma_clk = issue * 2.0 * rows_per_cta * n_eff * block_k / flop_rate;  // per SM
    // calibration on M = 192..256, N = K = 8192: a K block of a 128-column tile took 471 cycles on one
    // CTA and 415 on a pair, where the line above says 522 and 563
    if (tile_n < 256) mma_clk *= (cta_group == 2) ? 0.74 : 0.90;
    const double fill_clk = (double(rows_per_cta) + double(tile_n) / cta_group) * 128.0 / kSmemFillBytesPerClkSm;
    // the ring must also cover the L2 -> shared-memory latency: (stages - 1) K blocks in flight
    const int stage_bytes = (rows_per_cta + tile_n / cta_group) * 128;
    const int stages = (200 * 1024) / stage_bytes;
    const double latency_clk = kLoadLatencyClk / double(stages > 1 ? stages - 1 : 1);
    double stage_clk = mma_clk > fill_clk ? mma_clk : fill_clk;
    if (latency_clk > stage_clk) stage_clk = latency_clk;
    // with two accumulators per CTA the epilogue does not overlap the next tile (measured about
    // 12 000 cycles per 256 x 256 bf16 tile, more for 4-byte results, less for the half-width
    // SwiGLU result); with one it hides behind the next tile's main loop
    double epilogue_clk = 0.0;
    if (rows_per_cta == 256) epilogue_clk = (kind == O64_KIND_S8) ? 20000.0 : (epi == EPI_SWIGLU ? 8000.0 : 12000.0);
    const double prologue_clk = 2500.0;  // first TMA round trip + epilogue tail of the last tile
    return (waves * (kblocks * stage_clk + epilogue_clk) + prologue_clk) / (kClockGHz * 1e6);
}

// Split-K of the one-CTA tile kernel: when a CTA-per-tile plan leaves most SMs idle and K is long,
// slices of K go to separate CTAs (the reference's cache model blocks K the same way when one level
// cannot hold a whole strip, osprey/be/lno/cache_model.cxx:6650-6727).  Measured on M x 8192 x 8192:
// worth it for few rows, not for M = 128 (the atomics grow with M).
static int auto_split_k(int64_t M, int64_t N, int64_t K, int tile_n, int tile_k, int num_ctas) {
    const long long tiles = ((M + 127) / 128) * ((N + tile_n - 1) / tile_n);
    const long long kblocks = (K + tile_k - 1) / tile_k;
    int sk = 1;
    if (tiles * 2 <= num_ctas && kblocks >= 16 && (M <= 64 || tiles * 8 <= num_ctas)) {
        sk = (int)(num_ctas / tiles);
        if (sk > kblocks / 8) sk = (int)(kblocks / 8);
        if (sk > 16) sk = 16;
        if (sk < 1) sk = 1;
    }
    return sk;
}

// O64_LNO="blocking_size=128x256x64:stages=4:cta_group=1:group_m=8:raster=0:num_ctas=148:split_k=1"
static void apply_env(o64_plan_t *pin) {
    const char *env = getenv("O64_LNO");
    if (!env || !*env) return;
    char buf[256];
    strncpy(buf, env, sizeof(buf) - 1);
    buf[sizeof(buf) - 1] = 0;
    for (char *tok = strtok(buf, ":"); tok; tok = strtok(nullptr, ":")) {
        int a, b, c;
        if (sscanf(tok, "blocking_size=%dx%dx%d", &a, &b, &c) == 3) {
            pin->tile_m = a;
            pin->tile_n = b;
            pin->tile_k = c;
        } else if (sscanf(tok, "stages=%d", &a) == 1) {
            pin->stages = a;
        } else if (sscanf(tok, "cta_group=%d", &a) == 1) {
            pin->cta_group = a;
        } else if (sscanf(tok, "group_m=%d", &a) == 1) {
            pin->group_m = a;
        } else if (sscanf(tok, "raster=%d", &a) == 1) {
            pin->raster = a;
        } else if (sscanf(tok, "num_ctas=%d", &a) == 1) {
            pin->num_ctas = a;
        } else if (sscanf(tok, "split_k=%d", &a) == 1) {
            pin->split_k = a;
        }
    }
}

void plan_choose(int kind, int epi, int64_t M, int64_t N, int64_t K, int num_sms,
                 const o64_plan_t *pin_in, o64_plan_t *out) {
    o64_plan_t pin;
    memset(&pin, 0, sizeof(pin));
    if (pin_in) pin = *pin_in;
    apply_env(&pin);

    memset(out, 0, sizeof(*out));
    out->kind = kind;
    const int eb = elem_bytes(kind);
    out->tile_k = 128 / eb;
    out->mma_k = 32 / eb;
    out->split_k = 1;
    out->num_ctas = (pin.num_ctas > 0 && pin.num_ctas <= num_sms) ? pin.num_ctas : num_sms;

    // candidates: (cta_group, tile_m) in {(1,128), (2,256), (2,512)} x tile_n in {256, 128};
    // pins remove candidates
    static const int kShapes[3][2] = {{2, 512}, {2, 256}, {1, 128}};
    int best_g = 0, best_n = 0, best_m = 0;
    double best_t = 1e300;
    for (int i = 0; i < 3; ++i) {
        const int g = kShapes[i][0], tm = kShapes[i][1];
        if (pin.cta_group && pin.cta_group != g) continue;
        if (g == 2 && out->num_ctas < 2) continue;
        if (pin.tile_m && pin.tile_m != tm) continue;
        if (tm > 128 && M <= tm / 2 && !pin.tile_m && !pin.cta_group) continue;  // half the rows would be padding
        for (int n = 256; n >= 128; n /= 2) {
            if (pin.tile_n && pin.tile_n != n) continue;
            if (tm == 512 && n != 256) continue;                      // not instantiated
            if (tm == 512 && epi > EPI_S32) continue;                 // the requantising tails: 128- and 256-row kernels only
            if (g == 2 && n == 128 && epi == EPI_SWIGLU) continue;  // not instantiated
            double t = predict_ms(kind, epi, M, N, K, n, out->num_ctas, g, tm);
            if (g == 1 && epi != EPI_SWIGLU && epi <= EPI_S32 && pin.split_k == 0) {
                // the one-CTA kernel may split K: the main loop shrinks, atomics and a finishing pass come on top
                const int sk = auto_split_k(M, N, K, n, out->tile_k, out->num_ctas);
                if (sk > 1) t = t / sk + 0.006;
            }
            if (t < best_t) {
                best_t = t;
                best_g = g;
                best_n = n;
                best_m = tm;
            }
        }
    }
    if (!best_g) {  // contradictory pins: fall back to the plain default
        best_g = 1;
        best_n = 256;
        best_m = 128;
    }
    out->cta_group = best_g;
    out->tile_m = best_m;
    out->mma_m = 128 * best_g;
    const int tile_n = best_n;
    out->tile_n = tile_n;
    out->mma_n = tile_n;
    out->stages = best_m == 512 ? 4 : (best_g == 2 ? ((tile_n == 256) ? 6 : 8) : ((tile_n == 256) ? 4 : 6));
    out->predicted_ms = predict_ms(kind, epi, M, N, K, tile_n, out->num_ctas, best_g, best_m);

    // L2 block: tiles are walked in groups of group_m tile rows.  Measured best on the 8192^3
    // GEMM: groups that span about 2048 rows of C (16 / 8 / 4 tiles of 128 / 256 / 512 rows).
    if (pin.group_m > 0) {
        out->group_m = pin.group_m;
    } else {
        out->group_m = 2048 / out->tile_m;
    }
    if (out->cta_group == 1 && epi != EPI_SWIGLU && epi <= EPI_S32) {
        const long long kblocks = (K + out->tile_k - 1) / out->tile_k;
        int sk = pin.split_k > 0 ? pin.split_k : auto_split_k(M, N, K, tile_n, out->tile_k, out->num_ctas);
        if (sk > kblocks) sk = (int)kblocks;
        out->split_k = sk;
        if (sk > 1 && pin.split_k <= 0) out->predicted_ms = out->predicted_ms / sk + 0.006;
    }
    out->raster = pin.raster ? 1 : 0;  // the automatic choice is 0 (M fastest)

    // Few rows of A against a large weight: bound by HBM.  The kernel for that case loads only the
    // rows of A that exist (16 / 32 / 64 / 128 per stage), which leaves room for more stages of
    // weight in flight, and gives each 128 x 256 tile to a cluster of S CTAs that split K and add
    // their partial sums through distributed shared memory.  Reported as split_k = -S.  A pinned
    // split_k of -1 asks for the kernel (S chosen), -2 / -4 / -8 fix S, >= 1 rules the kernel out.
    const bool skinny_pinned = pin.split_k < 0;
    const bool skinny_fits = M <= (skinny_pinned ? 512 : 128) && epi != EPI_SWIGLU && epi <= EPI_S32 && pin.cta_group != 2 &&
                             (pin.tile_m == 0 || pin.tile_m <= 128) && (pin.tile_n == 0 || pin.tile_n == 256 || pin.tile_n == 128);
    if (skinny_fits && (skinny_pinned || (pin.split_k == 0 && !pin.cta_group && !pin.tile_m && !pin.tile_n &&
                                          (double)N * (double)K * eb >= 2.0 * 1024 * 1024))) {
        const int a_rows = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
        // 128-column tiles halve the partial sums a CTA exchanges and double the tiles: measured
        // faster for more than 64 rows, and where 256-column tiles on clusters of 4 would leave
        // half of the SMs idle (more than 8 tiles; up to 8 take clusters of 8)
        const int64_t tiles256 = ((M + 127) / 128) * ((N + 255) / 256);
        int bn = pin.tile_n ? pin.tile_n : 256;
        if (!pin.tile_n && (M > 64 || (tiles256 > 8 && tiles256 * 8 <= out->num_ctas))) bn = 128;
        const int64_t tiles = ((M + 127) / 128) * ((N + bn - 1) / bn);
        const int64_t kbs = (K + out->tile_k - 1) / out->tile_k;
        int s = pin.split_k < -1 ? -pin.split_k : umma_skinny_split(M, N, K, eb, out->num_ctas, bn);
        if (s > bn / 32) s = bn / 32;
        if (s > kbs) s = 1;
        out->cta_group = 1;
        out->tile_m = a_rows;
        out->tile_n = bn;
        out->mma_m = 128;
        out->mma_n = bn;
        out->stages = (6 * (256 + 16) * 128) / ((bn + a_rows) * 128);
        if (out->stages > 8) out->stages = 8;
        out->group_m = 1;
        out->split_k = -s;
        const int ctas_used = (int)(tiles * s < out->num_ctas ? tiles * s : out->num_ctas);
        const double bytes = ((double)N * K + (double)M * K) * eb + (double)M * N * (kind == O64_KIND_S8 ? 4 : 2);
        const double hbm_ms = bytes / 6.5e9;  // measured copy bandwidth, about 6.5 TB/s
        // tensor pipe: every K block costs one 128 x 256 MMA group whatever M is
        const double block_k = 128.0 / eb;
        const double per_cta = double((tiles * kbs + ctas_used - 1) / ctas_used);
        const double mma_clk = 1.02 * 2.0 * 128.0 * bn * block_k / (kDenseBf16FlopPerClkSm * (eb == 1 ? 2.0 : 1.0));
        const double mma_ms = per_cta * mma_clk / (kClockGHz * 1e6);
        out->predicted_ms = (hbm_ms > mma_ms ? hbm_ms : mma_ms) + 0.005;
        out->num_ctas = ctas_used;
    }

    const char *tr = getenv("O64_TRACE");
    if (tr && strstr(tr, "plan")) {
        // after -LNO:verbose, "[i,j,k --> ... blocks k(128)[L1] outside i]" (osprey/be/lno/snl_test.cxx:918-954)
        fprintf(stderr,
                "[o64 plan kind=%d %lldx%lldx%lld --> tile %dx%dx%d (mma %dx%dx%d) stages=%d[SMEM] "
                "group_m=%d[L2] raster=%d ctas=%d cta_group=%d predicted=%.4f ms]\n",
                kind, (long long)M, (long long)N, (long long)K, out->tile_m, out->tile_n, out->tile_k,
                out->mma_m, out->mma_n, out->mma_k, out->stages, out->group_m, out->raster,
                out->num_ctas, out->cta_group, out->predicted_ms);
    }
}

}  // namespace o64
