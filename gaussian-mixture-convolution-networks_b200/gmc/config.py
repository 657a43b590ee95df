"""Package-wide constants (counterpart of the reference's src/gmc/config.py)."""
import os
import pathlib

source_dir = os.path.dirname(__file__)
data_base_path = pathlib.Path(f"{source_dir}/../../data")

# kept for API compatibility; the CUDA evaluation streams components and needs no slicing
eval_slize_size = 1024 * 1024 * 100
eval_img_n_sample_points = 50 * 50
