"""Cloud helpers (src/levanter/utils/cloud_utils.py:135-173).  The reference's TPU-VM shutdown calls have no counterpart on
a GPU node; what remains is writing to a local scratch directory and uploading once at the end."""
from __future__ import annotations

import contextlib
import shutil
import tempfile
from typing import Optional

from ..distributed import process_index, sync_global_devices  # noqa: F401  (the barrier taken before uploads is re-exported)


@contextlib.contextmanager
def temp_dir_before_upload(path: str, process_should_upload: Optional[bool] = None):
    """Yield a local directory; on exit copy its contents to ``path`` (any fsspec URL) from the uploading process (rank 0 by
    default) and delete the local copy."""
    if process_should_upload is None:
        process_should_upload = process_index() == 0
    tmp = tempfile.mkdtemp(prefix="lvb_upload_")
    try:
        yield tmp
        if process_should_upload:
            import fsspec

            fs, plain = fsspec.core.url_to_fs(path)
            fs.makedirs(plain, exist_ok=True)
            fs.put(tmp.rstrip("/") + "/", plain.rstrip("/") + "/", recursive=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def shutdown_tpu_vm(sleep_seconds: float = 300.0):
    """No TPU VM exists here; kept so that configs with ``shutdown_at_exit`` have something to call."""
    return None
