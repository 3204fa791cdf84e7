// The reference's kernels do not log; its host code (not compiled by the test oracle) does.
#pragma once
