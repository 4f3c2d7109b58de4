from .dynamic_resource_controller import (DefaultDynamicSchedulePolicy, DynamicResourceController,  # noqa: F401
                                          FixedRatioDynamicSchedulePolicy, StaticFullyAsyncPolicy)
