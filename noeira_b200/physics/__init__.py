from .model import (Actuator, Body, Geom, Joint, Options, RigidModel, half_cheetah, hopper, pendulum_cart,  # noqa: F401
                    planar_chain)
