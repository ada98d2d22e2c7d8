// TEST INFRASTRUCTURE ONLY: the reference header that includes this one is compiled for its
// declarations; nothing of the JSON library is used by the NF4 operator.
#pragma once
