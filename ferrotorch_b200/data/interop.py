"""Arrow and dataframe interop (ferrotorch-data/src/interop.rs:74-260): 1-D tensors <-> Arrow
arrays without a copy where the memory allows it, record batches / tables / dataframes of numeric
columns -> ``[rows, columns]`` tensors.  Nulls are an error: a tensor has no validity bitmap."""
from __future__ import annotations

import torch

_ARROW_TO_TORCH = {"float": torch.float32, "double": torch.float64, "halffloat": torch.float16, "int8": torch.int8,
                   "int16": torch.int16, "int32": torch.int32, "int64": torch.int64, "uint8": torch.uint8, "bool": torch.bool}


def tensor_to_arrow_array(tensor: torch.Tensor):
    """1-D CPU tensor -> ``pyarrow.Array`` (zero-copy for contiguous numeric tensors)."""
    import pyarrow as pa

    if tensor.dim() != 1:
        raise ValueError("tensor_to_arrow_array: expected a 1-D tensor, got shape %s" % (tuple(tensor.shape),))
    if tensor.dtype == torch.bfloat16:
        raise ValueError("tensor_to_arrow_array: Arrow has no bfloat16; convert to float32 first")
    return pa.array(tensor.detach().cpu().contiguous().numpy())


tensor_to_arrow_arrayref = tensor_to_arrow_array


def tensor_from_arrow_array(array, dtype: torch.dtype | None = None) -> torch.Tensor:
    """``pyarrow.Array`` / ``ChunkedArray`` of a primitive type without nulls -> 1-D tensor."""
    import pyarrow as pa

    if isinstance(array, pa.ChunkedArray):
        array = array.combine_chunks()
    if array.null_count:
        raise ValueError("tensor_from_arrow_array: the array holds %d nulls" % array.null_count)
    kind = str(array.type)
    if kind not in _ARROW_TO_TORCH:
        raise ValueError("tensor_from_arrow_array: unsupported Arrow type %s" % kind)
    np_arr = array.to_numpy(zero_copy_only=False)
    t = torch.from_numpy(np_arr.copy() if not np_arr.flags.writeable else np_arr)
    return t.to(dtype) if dtype is not None else t


def record_batch_to_tensor(batch, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``RecordBatch`` / ``Table`` with numeric columns of one length -> ``[rows, columns]``."""
    cols = [tensor_from_arrow_array(batch.column(i), dtype) for i in range(batch.num_columns)]
    if not cols:
        return torch.empty((batch.num_rows, 0), dtype=dtype)
    return torch.stack(cols, dim=1)


def dataframe_to_tensor(df, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """pandas (or any dataframe with ``to_numpy`` / a ``__dataframe__``-compatible ``to_arrow``)
    -> ``[rows, columns]``; non-numeric columns and missing values are errors."""
    if hasattr(df, "to_arrow") and not hasattr(df, "to_numpy"):
        return record_batch_to_tensor(df.to_arrow(), dtype)
    import numpy as np

    def numeric(dt) -> bool:
        try:
            return bool(np.issubdtype(dt, np.number)) or dt == bool
        except TypeError:                      # extension dtypes (strings, categories ...)
            return False

    bad = [str(c) for c in df.columns if not numeric(df[c].dtype)]
    if bad:
        raise ValueError("dataframe_to_tensor: non-numeric columns %s" % bad)
    if bool(df.isna().to_numpy().any()):
        raise ValueError("dataframe_to_tensor: the frame holds missing values")
    return torch.from_numpy(np.ascontiguousarray(df.to_numpy())).to(dtype)
