"""Readers and writers of the PINK binary files (data, SOM, mapping, rotation/flip) in Python.

Formats: FILE_FORMATS.md:53-85 of the reference; every file is an optional text header (lines starting with
'#', ended by '# END OF HEADER'), native-endian int32 fields and raw float32 data.  The C++ program
pink_b200/Pink reads and writes the same files (pink_b200/host/pink_files.hpp)."""
import numpy as np


def _split_header(raw):
    pos, lines = 0, []
    while pos < len(raw) and raw[pos:pos + 1] == b"#":
        end = raw.index(b"\n", pos) + 1
        lines.append(raw[pos:end])
        pos = end
        if lines[-1] == b"# END OF HEADER\n":
            break
    return b"".join(lines).decode(), pos


def _ints(raw, pos, n):
    return [int(v) for v in np.frombuffer(raw, np.int32, n, pos)], pos + 4 * n


def write_data_file(path, images, text_header=""):
    """images: (n, h, w) or (n, channels, h, w) float32."""
    images = np.ascontiguousarray(images, np.float32)
    dims = images.shape[1:]
    with open(path, "wb") as f:
        f.write(text_header.encode())
        np.array([2, 0, 0, images.shape[0], 0, len(dims)] + list(dims), np.int32).tofile(f)
        images.tofile(f)


def read_data_file(path):
    raw = open(path, "rb").read()
    header, pos = _split_header(raw)
    (version, ftype, dtype, entries, _layout, nd), pos = _ints(raw, pos, 6)
    dims, pos = _ints(raw, pos, nd)
    assert (version, ftype, dtype) == (2, 0, 0), "not a version 2 float data file"
    return np.frombuffer(raw, np.float32, entries * int(np.prod(dims)), pos).reshape([entries] + dims), header


def write_som_file(path, som, som_dims, text_header=""):
    """som: (n_neurons, [channels,] nd, nd) float32; som_dims: e.g. (10, 10) -- also for hexagonal maps."""
    som = np.ascontiguousarray(som, np.float32)
    ndims = som.shape[1:]
    with open(path, "wb") as f:
        f.write(text_header.encode())
        np.array([2, 1, 0, 0, len(som_dims)] + list(som_dims) + [0, len(ndims)] + list(ndims), np.int32).tofile(f)
        som.tofile(f)


def read_som_file(path):
    """Returns (som[n_neurons, ...neuron dims], som_dims, text_header)."""
    raw = open(path, "rb").read()
    header, pos = _split_header(raw)
    (version, ftype, dtype, _layout, sd), pos = _ints(raw, pos, 5)
    assert (version, ftype, dtype) == (2, 1, 0), "not a version 2 float SOM file"
    som_dims, pos = _ints(raw, pos, sd)
    (_nlayout, nd), pos = _ints(raw, pos, 2)
    ndims, pos = _ints(raw, pos, nd)
    data = np.frombuffer(raw, np.float32, -1, pos)
    return data.reshape([-1] + ndims), som_dims, header


def read_mapping_file(path):
    """Returns (distances[entries, n_neurons], som_dims)."""
    raw = open(path, "rb").read()
    _, pos = _split_header(raw)
    (version, ftype, _dtype, entries, _layout, sd), pos = _ints(raw, pos, 6)
    assert (version, ftype) == (2, 2), "not a version 2 mapping file"
    som_dims, pos = _ints(raw, pos, sd)
    return np.frombuffer(raw, np.float32, -1, pos).reshape(entries, -1), som_dims


def read_rot_flip_file(path):
    """Returns (flipped[entries, n_neurons] bool, angle[entries, n_neurons] float32 radians, som_dims)."""
    raw = open(path, "rb").read()
    _, pos = _split_header(raw)
    (version, ftype, entries, _layout, sd), pos = _ints(raw, pos, 5)
    assert (version, ftype) == (2, 3), "not a version 2 rotation file"
    som_dims, pos = _ints(raw, pos, sd)
    rec = np.frombuffer(raw, np.dtype([("flip", np.uint8), ("angle", "<f4")]), -1, pos)
    return rec["flip"].astype(bool).reshape(entries, -1), rec["angle"].reshape(entries, -1), som_dims
