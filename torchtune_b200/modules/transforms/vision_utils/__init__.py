from .geometry import find_supported_resolutions, get_canvas_best_fit, get_inscribed_size, pad_dim_to_size, resize, resize_with_pad, tile_crop

__all__ = ["find_supported_resolutions", "get_canvas_best_fit", "get_inscribed_size", "pad_dim_to_size", "resize", "resize_with_pad", "tile_crop"]
