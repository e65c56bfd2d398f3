// ref_dump runs the reference's own Pack / Unpack / MatVec / MatVecPackedBlob on seeded inputs and
// writes the results as one binary file, so that the C restatement in oracle/welvet_oracle.c can be
// pinned against the reference itself. It needs a Go toolchain and a checkout of
// github.com/openfluke/welvet; it is test infrastructure, never part of the product.
//
// Build and run from a checkout of the reference (this file copied or symlinked into it as
// cmd/ref_dump/main.go):
//
//	python tests/golden/make_ref_inputs.py                  # in this repository: writes tests/golden/ref_inputs.bin
//	go run ./cmd/ref_dump <ref_inputs.bin> <ref_go_dump.bin>   # in the reference checkout
//
// then place ref_go_dump.bin under tests/golden/ of this repository; tests/test_oracle.py picks it up.
//
// Input  (little endian): u32 ncases, then per case u32 format | u32 rows | u32 cols | f32 w[rows*cols] | f32 x[cols].
// Output (little endian): u32 ncases, then per case
//
//	u32 format | u32 rows | u32 cols | u32 blockWeights | u32 nraw | u32 nscales | u32 nmins | u32 hasSimd
//	raw[nraw] | f32 scales[nscales] | f32 mins[nmins] | f32 unpack[rows*cols] | f32 yScalar[rows] | f32 ySimd[rows]
//
// Calls made: quant.Pack (quant/pack.go:4-31), quant.Unpack (quant/unpack.go:4-34), quant.MatVec
// (quant/matvec.go:5-35), dense.MatVecPackedBlob (layers/dense/simd.go:571-614; only for rows that
// start on a 32-column boundary, where the SIMD drivers are defined).
package main

import (
	"bufio"
	"encoding/binary"
	"fmt"
	"io"
	"math"
	"os"

	"github.com/openfluke/welvet/layers/dense"
	"github.com/openfluke/welvet/quant"
)

func readU32(r io.Reader) uint32 {
	var v uint32
	if err := binary.Read(r, binary.LittleEndian, &v); err != nil {
		panic(err)
	}
	return v
}

func readF32s(r io.Reader, n int) []float32 {
	buf := make([]byte, 4*n)
	if _, err := io.ReadFull(r, buf); err != nil {
		panic(err)
	}
	out := make([]float32, n)
	for i := range out {
		out[i] = math.Float32frombits(binary.LittleEndian.Uint32(buf[4*i:]))
	}
	return out
}

func writeU32(w io.Writer, v uint32) {
	if err := binary.Write(w, binary.LittleEndian, v); err != nil {
		panic(err)
	}
}

func writeF32s(w io.Writer, v []float32) {
	buf := make([]byte, 4*len(v))
	for i, f := range v {
		binary.LittleEndian.PutUint32(buf[4*i:], math.Float32bits(f))
	}
	if _, err := w.Write(buf); err != nil {
		panic(err)
	}
}

func main() {
	if len(os.Args) != 3 {
		fmt.Fprintln(os.Stderr, "usage: ref_dump <ref_inputs.bin> <ref_go_dump.bin>")
		os.Exit(2)
	}
	in, err := os.Open(os.Args[1])
	if err != nil {
		panic(err)
	}
	defer in.Close()
	r := bufio.NewReader(in)
	outf, err := os.Create(os.Args[2])
	if err != nil {
		panic(err)
	}
	defer outf.Close()
	w := bufio.NewWriter(outf)
	defer w.Flush()

	n := int(readU32(r))
	writeU32(w, uint32(n))
	for c := 0; c < n; c++ {
		format := quant.Format(readU32(r))
		rows, cols := int(readU32(r)), int(readU32(r))
		wts := readF32s(r, rows*cols)
		x := readF32s(r, cols)
		b, err := quant.Pack(format, wts, rows, cols)
		if err != nil {
			panic(fmt.Sprintf("case %d: Pack(%s, %dx%d): %v", c, format, rows, cols, err))
		}
		un, err := quant.Unpack(b)
		if err != nil {
			panic(fmt.Sprintf("case %d: Unpack: %v", c, err))
		}
		yScalar := make([]float32, rows)
		if err := quant.MatVec(b, x, yScalar); err != nil {
			panic(fmt.Sprintf("case %d: MatVec: %v", c, err))
		}
		ySimd := make([]float32, rows)
		hasSimd := uint32(0)
		if format != quant.FormatNone && cols%32 == 0 {
			if err := dense.MatVecPackedBlob(b, x, ySimd); err != nil {
				panic(fmt.Sprintf("case %d: MatVecPackedBlob: %v", c, err))
			}
			hasSimd = 1
		}
		writeU32(w, uint32(format))
		writeU32(w, uint32(rows))
		writeU32(w, uint32(cols))
		writeU32(w, uint32(b.BlockWeights))
		writeU32(w, uint32(len(b.Raw)))
		writeU32(w, uint32(len(b.Scales)))
		writeU32(w, uint32(len(b.Mins)))
		writeU32(w, hasSimd)
		if _, err := w.Write(b.Raw); err != nil {
			panic(err)
		}
		writeF32s(w, b.Scales)
		writeF32s(w, b.Mins)
		writeF32s(w, un[:rows*cols])
		writeF32s(w, yScalar)
		writeF32s(w, ySimd)
	}
}
