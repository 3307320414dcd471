// Tile schedule of the CTA-pair GEMM kernel: host and device see the same sequence.
#ifndef ROCWMMA_B200_CSRC_TILE_SCHEDULE_CUH
#define ROCWMMA_B200_CSRC_TILE_SCHEDULE_CUH
#include <cstdint>

namespace b200wmma
{
    // Which tiles a CTA pair works on, in which order (pair kernel).  The output is cut into
    // `wideCols` tile columns of width bn and, to their right, `tailCols` columns of width
    // bnTail.  Every pair takes the wide tiles p, p + P, p + 2P, ...  (P pairs); when their
    // number does not divide by P some pairs are one tile short -- up to a quarter of the run
    // on a 4096^2 output (256 tiles on 74 pairs).  The narrow tiles of the tail fill that gap:
    // the pairs that are short take two of them each first, the rest is dealt round-robin.
    // All three roles of both blocks of a pair call get() with i = 0, 1, 2, ... and see the
    // same sequence; the host uses the same code to compare schedules.
    //
    // Order of the wide tiles: band by band (a band = `band` tile rows whose rows of A stay in
    // L2), column by column inside a band.  With `snake` set, odd bands walk their columns
    // right to left, so a band starts on the columns of B the band before it touched last
    // and finds them in L2 (walking every band left to right streams all of B from DRAM
    // once per band: B is about as large as the L2).  With `mirror` set the whole sequence
    // runs backwards: a launch that mirrors its predecessor starts on the tiles -- and the
    // rows of A and columns of B -- that predecessor finished on.
    //
    // Split tiles.  When the last wave of a launch is less than half full, its `splitTiles`
    // tiles (the last ones in band order; wide tiles only, no tail columns) are each cut in
    // two along K and handed to two pairs: work item q < wideTiles - splitTiles is a whole
    // tile, the items after it come in twos, the halves of one tile.  getItem() reports the
    // half (`part`) and how many there are (`ways`: 1 or 2); the two halves meet in a
    // workspace (see the kernel).
    struct TileSchedule
    {
        uint32_t tilesM, wideCols, tailCols, bn, bnTail, band, pairs;
        uint32_t snake = 0, mirror = 0, splitTiles = 0;

        __host__ __device__ uint32_t wideTiles() const
        {
            return tilesM * wideCols;
        }
        __host__ __device__ uint32_t tailTiles() const
        {
            return tilesM * tailCols;
        }
        // wide tile t (band order, snake applied) -> tile row and first column
        __host__ __device__ void wideCoord(uint32_t t, uint32_t& tm, uint32_t& col0) const
        {
            const uint32_t perGroup = band * wideCols;
            const uint32_t group    = t / perGroup;
            const uint32_t firstM   = group * band;
            const uint32_t rows     = (tilesM - firstM) < band ? (tilesM - firstM) : band;
            const uint32_t r        = t % perGroup;
            const uint32_t col      = r / rows;
            tm                      = firstM + r % rows;
            col0 = ((snake && (group & 1u)) ? wideCols - 1u - col : col) * bn;
        }
        // i-th work item of pair p: tile row, first column, width, and which part of how many
        // along K (ways == 1: the whole tile).  `splitIndex` numbers the split tiles from 0.
        // false when the pair is done.
        __host__ __device__ bool getItem(uint32_t p, uint32_t i, uint32_t& tm, uint32_t& col0,
                                         uint32_t& width, uint32_t& part, uint32_t& ways,
                                         uint32_t& splitIndex) const
        {
            part       = 0u;
            ways       = 1u;
            splitIndex = 0u;
            if(splitTiles == 0u)
                return get(p, i, tm, col0, width);
            // split launches have no tail columns
            const uint32_t whole = wideTiles() - splitTiles;
            const uint32_t q     = p + i * pairs;
            if(q >= whole + 2u * splitTiles)
                return false;
            width = bn;
            if(q < whole)
            {
                wideCoord(mirror ? whole - 1u - q : q, tm, col0);
                return true;
            }
            splitIndex = (q - whole) / 2u;
            part       = (q - whole) % 2u;
            ways       = 2u;
            wideCoord(whole + splitIndex, tm, col0);
            return true;
        }
        // i-th tile of pair p: tile row, first column, width.  false when the pair is done.
        __host__ __device__ bool get(uint32_t p, uint32_t i, uint32_t& tm, uint32_t& col0,
                                     uint32_t& width) const
        {
            const uint32_t W = wideTiles(), T = tailTiles();
            const uint32_t base = W / pairs, nHi = W % pairs; // pairs [0, nHi) have base + 1
            const uint32_t mine = base + (p < nHi ? 1u : 0u);
            if(i < mine)
            {
                const uint32_t seq = p + i * pairs;
                wideCoord(mirror ? W - 1u - seq : seq, tm, col0);
                width = bn;
                return true;
            }
            i -= mine;
            // the pairs that are one wide tile short take two tail tiles each first
            const uint32_t nLo    = nHi == 0u ? 0u : pairs - nHi;
            const uint32_t bonus  = (2u * nLo) < T ? (2u * nLo) : T; // tail tiles dealt that way
            uint32_t       j      = 0xffffffffu;
            if(p >= nHi && nLo != 0u)
            {
                const uint32_t l  = p - nHi;
                const uint32_t my = (l < bonus ? 1u : 0u) + (l + nLo < bonus ? 1u : 0u);
                if(i < my)
                    j = l + i * nLo;
                else
                    i -= my;
            }
            if(j == 0xffffffffu)
            {
                const uint32_t rest = T - bonus;
                const uint32_t jj   = p + i * pairs;
                if(jj >= rest)
                    return false;
                j = bonus + jj;
            }
            tm    = j % tilesM;
            col0  = wideCols * bn + (j / tilesM) * bnTail;
            width = bnTail;
            return true;
        }
    };

} // namespace b200wmma
#endif
