"""Vision: camera capture, fiducial detection, pose and calibration (noeira/vision/)."""
from .camera import CameraReader, parse_camera_specs  # noqa: F401
from .calib import CameraCalib, calibrate_charuco, make_charuco_board, read_calib, write_calib  # noqa: F401
from .extrinsics import RigidFit, fit_rigid, fit_rigid_with_offset  # noqa: F401
from .preprocess import camera_frame_to_chw_rgb, pil_bilinear_u8, resize_pad  # noqa: F401
